"""Host-side drop-in logic (no GPU): the operator surface carries the reference's names and arities,
and install() wires them behind a stand-in for the reference's loader module."""
import inspect
import sys
import types

import pytest


def _reference_dir() -> str:
    """Where the reference project's sources are, if they are around: $GLQ_REFERENCE_DIR, else a folder named
    ``reference`` beside this repository."""
    import os
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    return os.environ.get("GLQ_REFERENCE_DIR") or os.path.join(os.path.dirname(here), "reference")


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
    ("fused_moe_grouped_gemm", 38), ("fused_moe_block_diag", 38),      # :203-246
    ("dequant_matvec", 8), ("dequant_matmul", 14),                     # :58-71
    ("input_rht", 8), ("output_rht", 7), ("output_rht_shards", 6),
])
def test_positional_arity_matches_reference_schema(name, arity):
    from glq_b200 import ops
    params = [p for p in inspect.signature(getattr(ops, name)).parameters.values()
              if p.name != "out_dtype" and p.kind == p.POSITIONAL_OR_KEYWORD]
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
    proxy = dropin.install(register_ops=False)
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


# ---------------------------------------------------------------------------------------------------
# torch.ops.glq registration: every served op exists, carries the reference's schema arity and has a
# fake (meta) implementation that yields the right shape / dtype without running a kernel
# ---------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def registered():
    import torch
    from glq_b200 import dropin
    names = dropin.register_torch_ops()
    assert sorted(names) == sorted(dropin.OPS)
    assert dropin.register_torch_ops() == names            # idempotent
    return torch.ops.glq


def test_every_served_op_is_registered_with_the_reference_arity(registered):
    from glq_b200 import dropin, ops
    for name, (schema, impl, fake) in dropin.OPS.items():
        op = getattr(registered, name)
        n_schema = len(op.default._schema.arguments)
        n_impl = len([p for p in inspect.signature(getattr(ops, name)).parameters.values()
                      if p.name != "out_dtype" and p.kind == p.POSITIONAL_OR_KEYWORD])
        assert n_schema == n_impl, name
        n_fake = inspect.signature(fake).parameters
        assert any(p.kind == p.VAR_POSITIONAL for p in n_fake.values()) or len(n_fake) == n_schema, name


def test_schemas_equal_the_reference_strings_when_the_reference_is_importable(registered):
    """Compares argument names and types with the strings in glq_vllm/custom_ops.py (read as text: the module
    itself needs vLLM's platform layer to import)."""
    import os
    import re
    path = os.path.join(_reference_dir(), "glq_vllm", "custom_ops.py")
    if not os.path.exists(path):
        pytest.skip("reference sources not present")
    from glq_b200 import dropin
    text = open(path).read()
    chunks = re.findall(r'\(\s*((?:"[^"]*"\s*)+)\)', text)
    ref = {}
    for c in chunks:
        joined = "".join(re.findall(r'"([^"]*)"', c))
        m = re.match(r"(\w+)(\(.*\)\s*->\s*(?:Tensor|\(\)))$", joined)
        if m:
            ref[m.group(1)] = m.group(2)
    norm = lambda t: re.sub(r"\s+", " ", t).strip()
    checked = 0
    for name, (schema, _, _) in dropin.OPS.items():
        assert name in ref, f"{name}: schema not found in the reference"
        assert norm(schema) == norm(ref[name]), name
        checked += 1
    assert checked == len(dropin.OPS)


def _fake_mode():
    from torch._subclasses.fake_tensor import FakeTensorMode
    return FakeTensorMode()


def test_fake_impls_give_shapes_and_dtypes(registered):
    import torch
    with _fake_mode():
        dev = "cuda"
        f16, i16, f32 = torch.float16, torch.int16, torch.float32
        B, n, m = 5, 576, 352
        x = torch.empty(B, n, dtype=f16, device=dev)
        sv, su = torch.empty(n, dtype=f16, device=dev), torch.empty(m, dtype=f16, device=dev)
        packed = torch.empty((m // 16) * (n // 16), 64, dtype=i16, device=dev)
        bl = torch.empty(2, dtype=torch.int64)
        meta = torch.empty(2, 4, dtype=torch.int32, device=dev)
        y = registered.fused_linear_trellis_3inst(x, sv, su, packed, bl, bl, meta, meta, 0.02, n, m, n, m)
        assert y.shape == (B, m) and y.dtype == f16 and y.device.type == "cuda"
        y = registered.fused_linear_trellis_3inst_rvq2(x, sv, su, packed, packed, bl, bl, meta, meta, 0.02, 0.2, n, m, n, m)
        assert y.shape == (B, m) and y.dtype == f16
        yr = torch.empty(B, 2 * m, dtype=f32, device=dev)
        assert registered.fused_linear_trellis_3inst_yrht(x, sv, packed, bl, meta, 0.02, n, n, m, yr, m) is None
        assert registered.fused_linear_trellis_3inst_yrht_rvq2(x, sv, packed, packed, bl, meta, 0.02, 0.2, n, n, m, yr, 0) is None
        out = torch.empty(B, 2 * m, dtype=f16, device=dev)
        assert registered.output_rht_shards(yr, torch.empty(2 * m, dtype=f16, device=dev), out, 2 * m, meta, 256) is None
        q = torch.empty(m, n // 8, dtype=i16, device=dev)
        cb = torch.empty(65536, 8, dtype=f16, device=dev)
        e_i, e_h = torch.empty(0, dtype=i16, device=dev), torch.empty(0, dtype=f16, device=dev)
        tail = (q, cb, 0.1, e_i, e_h, 0.0, e_i, e_h, 0.0)
        y = registered.fused_linear_block_diag(x, sv, su, q, cb, 0.02, n, m, n, m, bl, bl, meta, meta, *tail)
        assert y.shape == (B, m) and y.dtype == f16
        y = registered.fused_linear(x.new_empty(B, 512), sv.new_empty(512), su.new_empty(512),
                                    q.new_empty(512, 64), cb, 0.02, 500, 300, 512, 512, 9, 9, *tail)
        assert y.shape == (B, 300)
        xr = torch.empty(B, n, dtype=f16, device=dev)
        y = registered.dequant_matmul(xr, q, cb, 0.02, q, cb, 0.1, e_h, e_i, e_h, 0.0, e_i, e_h, 0.0)
        assert y.shape == (B, m) and y.dtype == f32
        y = registered.dequant_matvec(xr[0], q, cb, 0.02, q, cb, 0.1, e_h)
        assert y.shape == (m,) and y.dtype == f32
        buf = torch.empty(B, 1024, dtype=f32, device=dev)
        assert registered.input_rht(x, sv.new_empty(1024), buf, n, n, 1 / 32.0, 1024, 10) is None
        assert registered.output_rht(buf, su.new_empty(1024), out.new_empty(B, 1000), 1000, 1024, 10, 1 / 32.0) is None
        # MoE: (T, hidden) -> (T, hidden)
        E, T, H, I = 4, 7, 256, 128
        xm = torch.empty(T, H, dtype=f16, device=dev)
        ids = torch.empty(T, 2, dtype=torch.int64, device=dev)
        tw = torch.empty(T, 2, dtype=f32, device=dev)
        w13 = torch.empty(E, (2 * I // 16) * (H // 16), 64, dtype=i16, device=dev)
        w2 = torch.empty(E, (H // 16) * (I // 16), 64, dtype=i16, device=dev)
        s1 = torch.empty(E, 1, 1, dtype=i16, device=dev)
        vec = lambda k: torch.empty(k, dtype=f16, device=dev)
        sc = torch.empty(E, dtype=f32, device=dev)
        y = registered.fused_moe_trellis_3inst(xm, ids, tw, w13, s1, torch.empty(E, 2 * I, dtype=f16, device=dev), vec(H),
                                               sc, sc, w2, s1, torch.empty(E, H, dtype=f16, device=dev), vec(I), sc, sc,
                                               H, I, 2 * I, H, 2 * I, I, H, bl, bl, meta, meta, bl, bl, meta, meta, 1)
        assert y.shape == (T, H) and y.dtype == f16
        q13 = torch.empty(E, 2 * I, H // 8, dtype=i16, device=dev)
        q2 = torch.empty(E, H, I // 8, dtype=i16, device=dev)
        for op in (registered.fused_moe_grouped_gemm, registered.fused_moe_block_diag):
            y = op(xm, ids, tw, q13, torch.empty(E, 2 * I, dtype=f16, device=dev), vec(H), sc, q13, sc,
                   q2, torch.empty(E, H, dtype=f16, device=dev), vec(I), sc, q2, sc, cb, cb,
                   H, I, 2 * I, H, 2 * I, I, H, bl, bl, meta, meta, bl, bl, meta, meta, 0, s1, sc, s1, sc, cb)
            assert y.shape == (T, H) and y.dtype == f16


def test_reference_callers_bind_to_our_operator_signatures():
    """Runs the reference's own dispatch code (E8RHTLinear._trellis_linear_apply, glq/quantized_linear.py:838-899)
    against a recording stand-in for its extension module and binds the captured positional arguments to the
    functions of glq_b200.ops.  In a child process, so that ops registered by other tests cannot take the call."""
    import os
    import subprocess
    ref = _reference_dir()
    if not os.path.isdir(os.path.join(ref, "glq")):
        pytest.skip("reference sources not present")
    code = r"""
import inspect, sys, types
sys.path.insert(0, %r); sys.path.insert(0, %r)
import torch
from glq import inference_kernel as ik
from glq.quantized_linear import E8RHTLinear
from glq_b200 import dropin, ops
calls = []
class Rec:
    def __getattr__(self, name):
        if name not in dropin.SERVED:
            raise AttributeError(name)
        def f(*a):
            calls.append((name, a))
            return torch.zeros(a[0].shape[0], 32, dtype=torch.float16)
        return f
ik._glq_cuda, ik._cuda_ext_available = Rec(), True
x = torch.zeros(3, 64)
sv, su = torch.ones(64, dtype=torch.float16), torch.ones(32, dtype=torch.float16)
p = torch.zeros(8, 64, dtype=torch.int16)
bl = torch.tensor([64]); bm = torch.tensor([32]); e = torch.zeros(0, dtype=torch.float16)
meta = torch.zeros(1, 4, dtype=torch.int32)
E8RHTLinear._trellis_linear_apply(x, sv, su, p, e, bl, bm, meta, meta, 0.5, 64, 32, 64, 32)
E8RHTLinear._trellis_linear_apply(x, sv, su, p, e, bl, bm, meta, meta, 0.5, 64, 32, 64, 32,
                                  trellis_packed2=p, inv_resid_scale2=0.25)
assert [c[0] for c in calls] == ["glq_fused_linear_trellis_3inst_cuda", "glq_fused_linear_trellis_3inst_rvq2_cuda"], calls
for name, a in calls:
    b = inspect.signature(getattr(ops, name)).bind(*a)
    assert b.arguments["in_features"] == 64 and b.arguments["out_features"] == 32 and b.arguments["m_pad"] == 32
    assert b.arguments["wscale"] == 0.5
assert inspect.signature(ops.glq_fused_linear_trellis_3inst_rvq2_cuda).bind(*calls[1][1]).arguments["inv_resid_scale2"] == 0.25
print("bound", len(calls))
""" % (ref, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    env = dict(os.environ, TORCHDYNAMO_DISABLE="1")
    res = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=600)
    assert res.returncode == 0 and "bound 2" in res.stdout, res.stdout + res.stderr


def test_token_buckets_bound_the_number_of_plans():
    from glq_b200 import ops
    assert [ops.token_bucket(b) for b in (1, 8, 9, 64, 65, 128, 129, 300, 2048)] == [1, 8, 16, 64, 128, 128, 256, 512, 2048]
    assert all(ops.token_bucket(b) >= b for b in range(1, 5000))
    assert len({ops.token_bucket(b) for b in range(1, 2049)}) <= 24


def test_device_status_surfaces_as_an_error(monkeypatch):
    """A non-zero status word (a kernel that gave up on a bounded wait) must reach the caller as a
    RuntimeError carrying GLQB_E_DEVICE; made on the host with a stand-in for the library."""
    from glq_b200 import _lib, ops, plan

    class FakeLib:
        def glqb_plan_status(self, handle, out):
            out._obj.value = 3
            return -4
        def glqb_last_error(self):
            return b"a kernel gave up waiting (status 3): results of that run are invalid"
        def glqb_plan_destroy(self, handle):
            pass
    fake = FakeLib()
    monkeypatch.setattr(_lib, "_lib", fake)
    p = plan.Plan.__new__(plan.Plan)
    p.lib, p.handle = fake, 1
    monkeypatch.setitem(ops._PLAN_CACHE, ("fake",), p)
    with pytest.raises(RuntimeError, match=r"code -4.*gave up"):
        ops.check_device_status()
    p.handle = None
