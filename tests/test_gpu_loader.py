"""Loader-side glue (glq_b200/loader.py) end to end on the GPU: a small checkpoint is written to disk, read back
through the checkpoint reader, loaded into layers with the four calls a serving framework makes
(create_weights, the weight loader, process_weights_after_loading, apply) and compared with the oracle."""
from __future__ import annotations

import json
import os
import types

import numpy as np
import pytest
import torch

from glq_b200 import checkpoint as ck
from oracle import c_oracle as CO
from oracle import glq_oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-3
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def relerr(y, ref):
    y, ref = np.asarray(y, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    return np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30)


def _signs(rng, n):
    return (rng.integers(0, 2, size=n) * 2 - 1).astype(np.float16)


def _trellis(rng, m, n, sv, k=4, k2=0):
    d = {"trellis_packed": rng.integers(0, 65536, size=((m // 16) * (n // 16), 16 * k), dtype=np.uint16).view(np.int16),
         "SU": _signs(rng, m), "SV": sv, "Wscale": np.float32(0.01 + 0.02 * rng.random())}
    W = CO.trellis_decode(d["trellis_packed"], m, n, k).astype(np.float32)
    if k2:
        d["trellis_packed2"] = rng.integers(0, 65536, size=((m // 16) * (n // 16), 16 * k2), dtype=np.uint16).view(np.int16)
        d["inv_resid_scale2"] = np.float32(0.125)
        W = W + CO.trellis_decode(d["trellis_packed2"], m, n, k2).astype(np.float32) * np.float32(0.125)
    return d, W


def _write(folder, layers, config):
    tensors = {f"{p}.{k}": torch.from_numpy(np.asarray(v)) for p, d in layers.items() for k, v in d.items()}
    ck.write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    with open(os.path.join(folder, "quantize_config.json"), "w") as f:
        json.dump(config, f)


def test_trellis_checkpoint_through_the_loader(tmp_path):
    from glq_b200 import ops
    from glq_b200.loader import LinearMethod
    rng = np.random.default_rng(11)
    n, sizes = 576, [352, 96, 96]
    sv = _signs(rng, n)
    parts = [_trellis(rng, m, n, sv) for m in sizes]                       # q/k/v: separately quantized, one SV (same seed)
    down, W_down = _trellis(rng, 128, 352, _signs(rng, 352), 4, 2)         # a 6 bpw layer stored whole
    base = "model.layers.0."
    layers = {base + f"self_attn.{p}_proj": d for p, (d, _) in zip("qkv", parts)}
    layers[base + "mlp.down_proj"] = down
    _write(str(tmp_path), layers, {"bpw": 4, "codebook": "trellis", "variant": "3inst", "trellis_layout": "kernel",
                                   "layer_bpw": {**{base + f"self_attn.{p}_proj": 4 for p in "qkv"}, base + "mlp.down_proj": 6}})
    c = ck.Checkpoint(str(tmp_path))
    assert len(c.validate()) == 4
    method = LinearMethod(c.config)
    assert c.config.bpw_of("model.layers.0.self_attn.qkv_proj") == 4

    qkv = types.SimpleNamespace()
    method.create_weights(qkv, n, sizes, n, sum(sizes), torch.bfloat16)
    method.load_from(qkv, c, [base + f"self_attn.{p}_proj" for p in "qkv"])
    with pytest.raises(RuntimeError, match="process_weights_after_loading"):
        method.apply(qkv, torch.zeros(1, n, device="cuda", dtype=torch.bfloat16))
    method.process_weights_after_loading(qkv)
    assert qkv.glq_shared_sv
    for B in (1, 5, 40):
        x = torch.from_numpy(rng.standard_normal((B, n)).astype(np.float32)).cuda().to(torch.bfloat16)
        y = method.apply(qkv, x)
        assert y.shape == (B, sum(sizes)) and y.dtype == torch.bfloat16
        xf = x.float().cpu().numpy()
        ref = np.concatenate([O.linear_forward(xf, W, d["SU"], sv, float(d["Wscale"])) for d, W in parts], axis=1)
        assert relerr(y.float().cpu().numpy(), ref) <= TOL + 2.0 ** -8, B

    dn = types.SimpleNamespace()
    method6 = LinearMethod(c.config, bpw=6)
    method6.create_weights(dn, 352, [128], 352, 128, torch.float16)
    for name in ("trellis_packed", "trellis_packed2", "inv_resid_scale2", "SU", "SV", "Wscale"):
        method6.load_weight(dn, name, c.tensor(base + "mlp.down_proj." + name))
    method6.process_weights_after_loading(dn)
    x = torch.from_numpy(rng.standard_normal((3, 7, 352)).astype(np.float32)).cuda().half()
    bias = torch.randn(128, device="cuda", dtype=torch.float16)
    y = method6.apply(dn, x, bias)
    assert y.shape == (3, 7, 128)
    ref = O.linear_forward(x.float().cpu().numpy().reshape(21, 352), W_down, down["SU"], down["SV"], float(down["Wscale"]))
    assert relerr((y - bias).float().cpu().numpy().reshape(21, 128), ref) <= TOL + 2.0 ** -10
    c.close()
    ops.clear_caches()


def test_e8_checkpoint_through_the_loader(tmp_path):
    from glq_b200 import ops
    from glq_b200.loader import LinearMethod
    rng = np.random.default_rng(12)
    table = np.load(os.path.join(ROOT, "glq_b200", "data", "e8_shell_packed.npy"))
    cb = torch.from_numpy(O.e8_unpack_table(table).astype(np.float16))
    m, n = 320, 576                                                        # not powers of two: block-diagonal layer
    q = [rng.integers(0, 65536, size=(m, n // 8), dtype=np.uint16).view(np.int16) for _ in range(2)]
    su, sv = _signs(rng, m), _signs(rng, n)
    layer = {"Qidxs": q[0], "Qidxs2": q[1], "inv_resid_scale": np.float32(0.1), "SU": su, "SV": sv, "Wscale": np.float32(0.02)}
    _write(str(tmp_path), {"lm.layers.3.mlp.up_proj": layer}, {"bpw": 4, "codebook": "e8_shell"})
    c = ck.Checkpoint(str(tmp_path))
    info = c.validate()["lm.layers.3.mlp.up_proj"]
    assert info.n_stages == 2 and info.block_diagonal
    method = LinearMethod(c.config, codebook=cb, codebook2=cb)
    up = types.SimpleNamespace()
    method.create_weights(up, n, [m], n, m, torch.bfloat16)
    method.load_from(up, c, ["lm.layers.3.mlp.up_proj"])
    method.process_weights_after_loading(up)
    W = CO.e8_decode(q, [table, table], [0.1], m, n)
    for B in (1, 17):
        x = torch.from_numpy(rng.standard_normal((B, n)).astype(np.float32)).cuda().to(torch.bfloat16)
        y = method.apply(up, x)
        ref = O.linear_forward(x.float().cpu().numpy(), W, su, sv, 0.02)
        assert relerr(y.float().cpu().numpy(), ref) <= TOL + 2.0 ** -8, B
    c.close()
    ops.clear_caches()


def test_refusals():
    from glq_b200.loader import LinearMethod
    cfg = ck.QuantizeConfig.from_dict({"bpw": 4, "codebook": "trellis", "variant": "3inst", "trellis_layout": "kernel"})
    method = LinearMethod(cfg)
    layer = types.SimpleNamespace()
    with pytest.raises(ck.CheckpointError, match="32 x 32"):
        method.create_weights(layer, 2048, [1376 // 2 + 8], 2048, 696, torch.bfloat16)      # a shard that cuts a group
    method.create_weights(layer, 64, [64], 64, 64, torch.bfloat16)
    with pytest.raises(ck.CheckpointError, match="does not belong"):
        method.load_weight(layer, "Qidxs", torch.zeros(64, 8, dtype=torch.int16))
    with pytest.raises(ck.CheckpointError, match="tlut"):
        method.load_weight(layer, "tlut", torch.zeros(512, 2, dtype=torch.float16))
    with pytest.raises(ck.CheckpointError, match="codebook table"):
        LinearMethod(ck.QuantizeConfig.from_dict({"codebook": "e8_shell"}))
