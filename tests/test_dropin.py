"""Host-side drop-in logic (no GPU): the operator surface carries the reference's names and arities,
and install() wires them behind a stand-in for the reference's loader module."""
import inspect
import sys
import types

import pytest


def test_ops_module_exports_reference_names():
    from glq_b200 import dropin, ops
    for name in dropin.SERVED:
        assert callable(getattr(ops, name)), name


@pytest.mark.parametrize("name,arity", [
    ("fused_linear_trellis_3inst", 13),          # glq_vllm/custom_ops.py:373-378
    ("fused_linear_trellis_3inst_rvq2", 15),     # :402-407
    ("fused_linear_trellis_3inst_yrht", 11),     # :388-392
    ("fused_linear_trellis_3inst_yrht_rvq2", 13),
    ("fused_linear", 21),                        # :105-112
    ("fused_linear_block_diag", 23),             # :118-126
    ("fused_moe_trellis_3inst", 31),             # :22-36
    ("input_rht", 8), ("output_rht", 7), ("output_rht_shards", 6),
])
def test_positional_arity_matches_reference_schema(name, arity):
    from glq_b200 import ops
    params = [p for p in inspect.signature(getattr(ops, name)).parameters.values() if p.name != "out_dtype"]
    assert len(params) == arity


def test_install_injects_proxy_into_reference_loader(monkeypatch):
    from glq_b200 import dropin
    glq = types.ModuleType("glq")
    ik = types.ModuleType("glq.inference_kernel")
    ik._glq_cuda, ik._cuda_ext_available = None, False
    glq.inference_kernel = ik
    monkeypatch.setitem(sys.modules, "glq", glq)
    monkeypatch.setitem(sys.modules, "glq.inference_kernel", ik)
    monkeypatch.setitem(sys.modules, "glq_vllm.custom_ops", None)
    proxy = dropin.install(register_torch_ops=False)
    assert ik._cuda_ext_available is True and ik._glq_cuda is proxy
    assert hasattr(proxy, "glq_fused_linear_trellis_3inst_rvq2_cuda")
    assert not hasattr(proxy, "glq_fused_linear_e8p_cuda")        # unserved formats stay absent


def test_linear_module_buffers_match_reference_layout():
    from glq_b200.linear import GLQLinear
    l = GLQLinear(48, 32)
    assert l.Qidxs.shape == (32, 8) and l.SU.shape == (32,) and l.SV.shape == (64,) and l.Wscale.shape == ()
    assert (l.m_pad, l.n_pad) == (32, 64)
    l = GLQLinear(50, 33)
    assert (l.m_pad, l.n_pad) == (64, 64)
    t = GLQLinear(576, 352, codebook_type="trellis")
    assert t.blocks_n == [512, 64] and t.blocks_m == [256, 64, 32] and t.trellis_packed.numel() == 0
    import torch
    with pytest.raises(RuntimeError):
        t(torch.zeros(1, 576))                                      # CPU tensor: no fallback
