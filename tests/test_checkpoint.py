"""Checkpoint side of the boundary (glq_b200/checkpoint.py), on CPU: the safetensors reader against the
installed safetensors package, the config rules the reference's serving config enforces
(glq_vllm/config.py:30-47, 75-121), the [gate; up] split (glq/quantize_model.py:654-677) against the oracle's
decode, and the per-layer storage checks."""
from __future__ import annotations

import json
import os

import numpy as np
import pytest
import torch

from glq_b200 import checkpoint as ck
from oracle import glq_oracle as O


def _trellis_layer(rng, m, n, k=4, k2=0):
    d = {"trellis_packed": torch.from_numpy(rng.integers(0, 65536, size=((m // 16) * (n // 16), 16 * k), dtype=np.uint16).view(np.int16)),
         "SU": torch.from_numpy((rng.integers(0, 2, size=m) * 2 - 1).astype(np.float16)),
         "SV": torch.from_numpy((rng.integers(0, 2, size=n) * 2 - 1).astype(np.float16)),
         "Wscale": torch.tensor(0.02, dtype=torch.float32)}
    if k2:
        d["trellis_packed2"] = torch.from_numpy(rng.integers(0, 65536, size=((m // 16) * (n // 16), 16 * k2), dtype=np.uint16).view(np.int16))
        d["inv_resid_scale2"] = torch.tensor(0.1, dtype=torch.float32)
    return d


def _e8_layer(rng, m, n, stages=2):
    d = {"Qidxs": torch.from_numpy(rng.integers(0, 65536, size=(m, n // 8), dtype=np.uint16).view(np.int16)),
         "SU": torch.from_numpy((rng.integers(0, 2, size=m) * 2 - 1).astype(np.float16)),
         "SV": torch.from_numpy((rng.integers(0, 2, size=n) * 2 - 1).astype(np.float16)),
         "Wscale": torch.tensor(0.02, dtype=torch.float32)}
    for s in range(1, stages):
        d[f"Qidxs{s + 1}"] = torch.from_numpy(rng.integers(0, 65536, size=(m, n // 8), dtype=np.uint16).view(np.int16))
        d["inv_resid_scale" if s == 1 else f"inv_resid_scale{s}"] = torch.tensor(0.1 ** s, dtype=torch.float32)
    return d


def test_safetensors_round_trip_and_agreement_with_the_package(tmp_path):
    rng = np.random.default_rng(0)
    tensors = {"a.SU": torch.from_numpy(rng.standard_normal(7).astype(np.float16)),
               "a.Qidxs": torch.from_numpy(rng.integers(-32768, 32767, size=(5, 3), dtype=np.int16)),
               "b.weight": torch.randn(4, 6).to(torch.bfloat16), "scalar": torch.tensor(1.5), "empty": torch.zeros(0, dtype=torch.int16),
               "i64": torch.arange(5)}
    p = str(tmp_path / "x.safetensors")
    ck.write_safetensors(p, tensors, metadata={"format": "pt"})
    back = ck.read_safetensors(p)
    assert set(back) == set(tensors)
    for k in tensors:
        assert back[k].dtype == tensors[k].dtype and back[k].shape == tensors[k].shape and torch.equal(back[k], tensors[k]), k
    st = pytest.importorskip("safetensors.torch")
    theirs = st.load_file(p)                       # our writer read by the package
    for k in tensors:
        assert torch.equal(theirs[k], tensors[k]), k
    p2 = str(tmp_path / "y.safetensors")
    st.save_file({k: v.contiguous() for k, v in tensors.items()}, p2)
    ours = ck.read_safetensors(p2)                 # the package's file read by our reader
    for k in tensors:
        assert torch.equal(ours[k], tensors[k]), k


def test_safetensors_rejects_damaged_files(tmp_path):
    p = str(tmp_path / "x.safetensors")
    ck.write_safetensors(p, {"t": torch.arange(10, dtype=torch.int32)})
    raw = open(p, "rb").read()
    open(p, "wb").write(raw[:-4])                  # truncated data
    with pytest.raises(ck.CheckpointError, match="byte range"):
        ck.SafetensorsFile(p)
    open(p, "wb").write(b"\xff" * 8 + raw[8:])     # absurd header length
    with pytest.raises(ck.CheckpointError, match="header length"):
        ck.SafetensorsFile(p)
    open(p, "wb").write(raw[:3])
    with pytest.raises(ck.CheckpointError, match="shorter"):
        ck.SafetensorsFile(p)


def test_config_rules():
    ok = ck.QuantizeConfig.from_dict({"bpw": 4, "codebook": "trellis", "variant": "3inst", "trellis_layout": "kernel"})
    assert ok.bpw == 4 and ok.block_diagonal
    with pytest.raises(ck.CheckpointError, match="natural"):
        ck.QuantizeConfig.from_dict({"codebook": "trellis", "variant": "3inst"})
    with pytest.raises(ck.CheckpointError, match="no kernel"):
        ck.QuantizeConfig.from_dict({"codebook": "trellis", "variant": "bitshift", "trellis_layout": "kernel"})
    with pytest.raises(ck.CheckpointError, match="HYB"):
        ck.QuantizeConfig.from_dict({"codebook": "trellis", "trellis_layout": "kernel"})       # default variant hyb
    with pytest.raises(ck.CheckpointError, match="E8P"):
        ck.QuantizeConfig.from_dict({"codebook": "e8p"})
    assert ck.QuantizeConfig.from_dict({}).codebook == "e8_shell"


def test_layer_rate_lookup_follows_renamed_and_merged_layers():
    c = ck.QuantizeConfig.from_dict({"bpw": 2, "layer_bpw": {
        "model.language_model.layers.0.self_attn.q_proj": 3, "model.language_model.layers.0.self_attn.k_proj": 4,
        "model.language_model.layers.0.self_attn.v_proj": 2, "model.layers.1.mlp.down_proj": 4}})
    assert c.bpw_of("model.layers.1.mlp.down_proj") == 4
    assert c.bpw_of("model.layers.0.self_attn.qkv_proj") == 4                  # merged: the largest of its parts
    assert c.bpw_of("language_model.model.layers.0.self_attn.q_proj") == 3     # multimodal renaming
    assert c.bpw_of("model.layers.0.mlp.gate_up_proj") is None                 # not in the table: not quantized
    assert ck.QuantizeConfig.from_dict({"bpw": 3}).bpw_of("anything") == 3     # no table: the global rate


def test_gate_up_split_matches_decoding_the_joint_layer():
    rng = np.random.default_rng(3)
    n, gate, up = 64, 64, 96
    joint = _trellis_layer(rng, gate + up, n, 3)["trellis_packed"]
    g, u = ck.split_trellis_packed(joint, gate, up, n)
    W = O.trellis_decode_layer(joint.numpy(), gate + up, n, 3)
    assert np.array_equal(O.trellis_decode_layer(g.numpy(), gate, n, 3), W[:gate])
    assert np.array_equal(O.trellis_decode_layer(u.numpy(), up, n, 3), W[gate:])
    with pytest.raises(ck.CheckpointError, match="multiples of 32"):
        ck.split_trellis_packed(joint, 80, 80, n)
    with pytest.raises(ck.CheckpointError, match="tiles expected"):
        ck.split_trellis_packed(joint, 64, 64, n)


def test_trellis_rates():
    assert [ck.trellis_rates(b) for b in (2, 4, 5, 8)] == [(2, 0), (4, 0), (4, 1), (4, 4)]
    with pytest.raises(ck.CheckpointError):
        ck.trellis_rates(9)


def test_validate_layer_reads_dimensions_and_names_the_bad_buffer():
    rng = np.random.default_rng(4)
    t = _trellis_layer(rng, 96, 64, 4, 2)
    info = ck.validate_layer(t, "trellis")
    assert (info.m_pad, info.n_pad, info.n_stages, info.bits) == (96, 64, 2, (4, 2))
    assert info.code_bytes == 96 * 64 * 6 // 8
    e = _e8_layer(rng, 24, 40, 3)
    info = ck.validate_layer(e, "e8_shell")
    assert (info.m_pad, info.n_pad, info.n_stages, info.block_diagonal) == (24, 40, 3, True)
    assert ck.validate_layer(_e8_layer(rng, 32, 64, 1), "e8_shell").block_diagonal is False      # powers of two: legacy padding
    bad = dict(t); bad["SU"] = bad["SU"].clone(); bad["SU"][3] = 0.5
    with pytest.raises(ck.CheckpointError, match="SU holds values"):
        ck.validate_layer(bad, "trellis")
    bad = dict(t); bad["trellis_packed"] = bad["trellis_packed"][:-1]
    with pytest.raises(ck.CheckpointError, match="trellis_packed"):
        ck.validate_layer(bad, "trellis")
    bad = dict(t); bad["inv_resid_scale2"] = torch.tensor(0.0)
    with pytest.raises(ck.CheckpointError, match="inv_resid_scale2"):
        ck.validate_layer(bad, "trellis")
    bad = dict(t); bad["tlut"] = torch.zeros(512, 2, dtype=torch.float16)
    with pytest.raises(ck.CheckpointError, match="tlut"):
        ck.validate_layer(bad, "trellis")
    bad = dict(e); bad["Qidxs2"] = bad["Qidxs2"][:, :-1]
    with pytest.raises(ck.CheckpointError, match="Qidxs2"):
        ck.validate_layer(bad, "e8_shell")
    bad = dict(e); del bad["Wscale"]
    with pytest.raises(ck.CheckpointError, match="Wscale"):
        ck.validate_layer(bad, "e8_shell")


def test_checkpoint_folder_index_and_validation(tmp_path):
    rng = np.random.default_rng(5)
    layers = {"model.layers.0.self_attn.q_proj": _trellis_layer(rng, 64, 64, 4), "model.layers.0.mlp.down_proj": _trellis_layer(rng, 64, 96, 4, 1)}
    a = {f"{p}.{k}": v for p, d in list(layers.items())[:1] for k, v in d.items()}
    b = {f"{p}.{k}": v for p, d in list(layers.items())[1:] for k, v in d.items()}
    a["model.norm.weight"] = torch.ones(64, dtype=torch.bfloat16)
    ck.write_safetensors(str(tmp_path / "model-00001-of-00002.safetensors"), a)
    ck.write_safetensors(str(tmp_path / "model-00002-of-00002.safetensors"), b)
    (tmp_path / "quantize_config.json").write_text(json.dumps(
        {"bpw": 4, "codebook": "trellis", "variant": "3inst", "trellis_layout": "kernel",
         "layer_bpw": {"model.layers.0.self_attn.q_proj": 4, "model.layers.0.mlp.down_proj": 5}}))
    c = ck.Checkpoint(str(tmp_path))
    assert sorted(c.layers) == sorted(layers)
    infos = c.validate()
    assert infos["model.layers.0.mlp.down_proj"].bits == (4, 1)
    lin = c.load_linear("model.layers.0.mlp.down_proj")
    assert (lin.in_features, lin.out_features) == (96, 64)
    assert torch.equal(lin.trellis_packed2, layers["model.layers.0.mlp.down_proj"]["trellis_packed2"])
    c.close()
    # a rate in the config that the stored bit-streams contradict
    (tmp_path / "quantize_config.json").write_text(json.dumps(
        {"bpw": 3, "codebook": "trellis", "variant": "3inst", "trellis_layout": "kernel"}))
    c = ck.Checkpoint(str(tmp_path))
    with pytest.raises(ck.CheckpointError, match="bpw"):
        c.validate()
    c.close()


def test_loader_takes_the_rank_s_own_shard_buffers_when_the_checkpoint_has_them():
    """Host logic of the tensor-parallel loader (no GPU): with a communicator of G ranks the loader prefers the
    buffers stored under <layer>.tp<G>.<rank>.<buffer>, and falls back to the whole layer otherwise."""
    import types
    from glq_b200.loader import LinearMethod, tp_buffer_key
    rng = np.random.default_rng(6)
    cfg = ck.QuantizeConfig.from_dict({"bpw": 4, "codebook": "trellis", "variant": "3inst", "trellis_layout": "kernel"})
    whole = _trellis_layer(rng, 64, 128, 4)
    shard1 = _trellis_layer(rng, 64, 64, 4)
    tensors = {f"m.o_proj.{k}": v for k, v in whole.items()}
    tensors.update({tp_buffer_key("m.o_proj", k, 2, 1): v for k, v in shard1.items()})
    fake_comm = types.SimpleNamespace(world=2, rank=1)
    layer = types.SimpleNamespace()
    m = LinearMethod(cfg, comm=fake_comm)
    m.create_weights(layer, 64, [64], 128, 64, torch.bfloat16, row_parallel=True)
    m.load_from(layer, tensors, ["m.o_proj"])
    assert layer.glq_tp_sharded and layer.glq_row_parallel
    assert torch.equal(layer.glq_buffers["trellis_packed"].get_shard(0), shard1["trellis_packed"])
    # rank 0 has no shard of its own in this checkpoint: the whole layer is taken
    layer0 = types.SimpleNamespace()
    m0 = LinearMethod(cfg, comm=types.SimpleNamespace(world=2, rank=0))
    m0.create_weights(layer0, 128, [64], 128, 64, torch.bfloat16, row_parallel=True)
    m0.load_from(layer0, tensors, ["m.o_proj"])
    assert not layer0.glq_tp_sharded
    assert torch.equal(layer0.glq_buffers["SV"].get_shard(0), whole["SV"])
    with pytest.raises(ck.CheckpointError, match="shards"):
        m0.load_from(layer0, tensors, ["a", "b"])
