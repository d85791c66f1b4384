"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle and the reference's
golden outputs.  Bit-exact for decode dumps; layer outputs within max|err| / max|ref| <= 2e-3 (the
tolerance the target states for fp16-operand / fp32-accumulate kernels with bf16 or fp16 output)."""
import numpy as np
import pytest
import torch

from oracle import glq_oracle as O

pytestmark = pytest.mark.gpu

TOL = 2e-3
# A 16-bit result cannot be closer to an fp32 reference than half a unit in its last place:
# 2^-8 of the value for bf16, 2^-11 for fp16.  The 2e-3 bound is asserted on fp32 results (what the
# kernels hold before the final rounding); 16-bit results get the rounding step added.
OUT_ROUND = {torch.float32: 0.0, torch.float16: 2.0 ** -11, torch.bfloat16: 2.0 ** -8}


def relerr(y, ref):
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30)


def cuda(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def signs(rng, n):
    return (rng.integers(0, 2, size=n) * 2 - 1).astype(np.float16)


def rand_packed(rng, m, n, K):
    return rng.integers(0, 65536, size=((m // 16) * (n // 16), 16 * K), dtype=np.uint16).view(np.int16)


@pytest.fixture(scope="module")
def ops():
    from glq_b200 import ops as _ops
    return _ops


@pytest.fixture(scope="module")
def e8_cb(e8_table):
    """fp16 CUDA codebook tensors (full and first-256) as the reference passes them to its ops."""
    full = cuda(e8_table.astype(np.float16))
    small = full[:256].contiguous()
    return full, small


# ---------------------------------------------------------------------------------------------
# decode dumps: bit exact
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("K", [1, 2, 3, 4])
@pytest.mark.parametrize("shape", [(32, 64), (64, 192), (96, 128)])
def test_trellis_dump_matches_reference_golden(ops, golden, K, shape):
    g = golden("golden_trellis.npz")
    m, n = shape
    key = f"K{K}_m{m}_n{n}"
    out = ops.glq_decompress_trellis_3inst_cuda(cuda(g[key + "_packed"]), m, n)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), g[key + "_dec"].view(np.uint16))


@pytest.mark.parametrize("K", [1, 2, 3, 4])
def test_trellis_dump_matches_oracle_large(ops, K):
    rng = np.random.default_rng(100 + K)
    m, n = 512, 2048
    packed = rand_packed(rng, m, n, K)
    out = ops.glq_decompress_trellis_3inst_cuda(cuda(packed), m, n).cpu().numpy()
    ref = O.trellis_decode_layer(packed, m, n, K)
    assert np.array_equal(out.view(np.uint16), ref.view(np.uint16))


@pytest.mark.parametrize("K2", [1, 2, 3, 4])
def test_trellis_two_stage_dump_bit_exact(ops, golden, K2):
    g = golden("golden_trellis.npz")
    key = f"rvq_K2_{K2}"
    out = ops.decompress_trellis_3inst_rvq2(cuda(g[key + "_p1"]), cuda(g[key + "_p2"]), float(g[key + "_inv"]), 64, 128)
    assert np.array_equal(out.cpu().numpy().view(np.uint32), g[key + "_dec"].view(np.uint32))


@pytest.mark.parametrize("stages", [1, 2, 3, 4])
def test_e8_dump_bit_exact(ops, e8_table, e8_cb, stages):
    rng = np.random.default_rng(stages)
    full, small = e8_cb
    m, n = 96, 320
    qs = [rng.integers(0, 65536, size=(m, n // 8), dtype=np.uint16).view(np.int16) for _ in range(stages)]
    inv = [1 / 3.0, 1 / 9.0, 1 / 27.0][:stages - 1]
    out = ops.dequant_e8([cuda(q) for q in qs], [full] * stages, inv).cpu().numpy()
    ref = O.e8_decode_nstage(qs, [e8_table] * stages, inv)
    assert np.array_equal(out.view(np.uint32), ref.view(np.uint32))


def test_e8_dump_small_second_table(ops, e8_table, e8_cb):
    rng = np.random.default_rng(9)
    full, small = e8_cb
    m, n = 64, 128
    q1 = rng.integers(0, 65536, size=(m, n // 8), dtype=np.uint16).view(np.int16)
    q2 = rng.integers(0, 256, size=(m, n // 8), dtype=np.uint16).view(np.int16)
    out = ops.dequant_e8([cuda(q1), cuda(q2)], [full, small], [0.25]).cpu().numpy()
    ref = O.e8_decode_nstage([q1, q2], [e8_table, e8_table[:256]], [0.25])
    assert np.array_equal(out.view(np.uint32), ref.view(np.uint32))


def test_e8_pack_table_matches_shipped(ops, e8_cb):
    import os
    full, _ = e8_cb
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    shipped = np.load(os.path.join(root, "glq_b200", "data", "e8_shell_packed.npy"))
    got = ops.e8_packed_table(full).cpu().numpy().view(np.uint32)
    assert np.array_equal(got, shipped)


# ---------------------------------------------------------------------------------------------
# trellis linears
# ---------------------------------------------------------------------------------------------
def _trellis_layer(rng, m, n, K, K2=0):
    p1 = rand_packed(rng, m, n, K)
    p2 = rand_packed(rng, m, n, K2) if K2 else None
    su, sv = signs(rng, m), signs(rng, n)
    wscale = float(np.float16(rng.uniform(0.5, 1.5) * 0.02))
    inv = 0.21 if K2 else 0.0
    if K2:
        W = O.trellis_decode_layer_nstage([p1, p2], [K, K2], [1.0, inv], m, n)
    else:
        W = O.trellis_decode_layer(p1, m, n, K).astype(np.float32)
    return p1, p2, su, sv, wscale, inv, W


def _run_trellis(ops, x_t, p1, p2, su, sv, wscale, inv, m, n, out_dtype=None):
    bn, bm = O.block_decompose(n), O.block_decompose(m)
    tn, tm = torch.tensor(bn), torch.tensor(bm)
    if p2 is None:
        return ops.fused_linear_trellis_3inst(x_t, cuda(sv), cuda(su), cuda(p1), tn, tm, None, None, wscale, n, m, n, m,
                                              out_dtype=out_dtype)
    return ops.fused_linear_trellis_3inst_rvq2(x_t, cuda(sv), cuda(su), cuda(p1), cuda(p2), tn, tm, None, None,
                                               wscale, inv, n, m, n, m, out_dtype=out_dtype)


@pytest.mark.parametrize("K,K2", [(2, 0), (3, 0), (4, 0), (4, 1), (4, 2), (4, 3), (4, 4)])
@pytest.mark.parametrize("B", [1, 5, 16, 33])
def test_trellis_linear_vs_oracle(ops, K, K2, B):
    rng = np.random.default_rng(K * 100 + K2 * 10 + B)
    m, n = 352, 576            # 256+64+32 rows, 512+64 columns: block-diagonal on both sides
    p1, p2, su, sv, wscale, inv, W = _trellis_layer(rng, m, n, K, K2)
    x = rng.standard_normal((B, n)).astype(np.float32)
    x_t = cuda(x, torch.bfloat16)
    ref = O.linear_forward(x_t.float().cpu().numpy(), W, su, sv, wscale)
    y32 = _run_trellis(ops, x_t, p1, p2, su, sv, wscale, inv, m, n, out_dtype=torch.float32)
    assert y32.dtype == torch.float32 and y32.shape == (B, m)
    assert relerr(y32.cpu().numpy(), ref) <= TOL
    y = _run_trellis(ops, x_t, p1, p2, su, sv, wscale, inv, m, n)
    assert y.dtype == torch.bfloat16 and y.shape == (B, m)
    assert torch.equal(y, y32.to(torch.bfloat16))     # the 16-bit result is the rounded fp32 result
    assert relerr(y.float().cpu().numpy(), ref) <= TOL + OUT_ROUND[torch.bfloat16]


@pytest.mark.parametrize("name", ["k2", "k3", "k4", "k4p2", "k4p4"])
def test_trellis_linear_vs_reference_golden(ops, golden, name):
    g = golden("golden_trellis_linear.npz")
    fin, fout, K, K2 = [int(v) for v in g[name + "_meta"]]
    p2 = g[name + "_packed2"] if K2 else None
    y = _run_trellis(ops, cuda(g[name + "_x"]), g[name + "_packed"], p2, g[name + "_SU"], g[name + "_SV"],
                     float(g[name + "_Wscale"]), float(g[name + "_inv_resid_scale2"]), fout, fin)
    assert y.dtype == torch.float32
    assert relerr(y.cpu().numpy(), g[name + "_y"]) <= TOL


@pytest.mark.parametrize("shape", [(2048, 2048), (512, 2048), (2048, 11008), (11008, 2048)])
def test_trellis_decode_shapes_b1(ops, shape):
    """Projection shapes of the decode benchmark (SmolLM3-3B), 4 bpw, batch 1."""
    m, n = shape
    rng = np.random.default_rng(m + n)
    p1, p2, su, sv, wscale, inv, W = _trellis_layer(rng, m, n, 4)
    x = rng.standard_normal((1, n)).astype(np.float32)
    x_t = cuda(x, torch.bfloat16)
    y = _run_trellis(ops, x_t, p1, None, su, sv, wscale, 0.0, m, n, out_dtype=torch.float32)
    ref = O.linear_forward(x_t.float().cpu().numpy(), W, su, sv, wscale)
    assert relerr(y.cpu().numpy(), ref) <= TOL
    y2 = _run_trellis(ops, x_t, p1, None, su, sv, wscale, 0.0, m, n, out_dtype=torch.float32)
    assert torch.equal(y, y2)          # deterministic


def test_trellis_row_parity_and_determinism(ops):
    """Row b of a batched call equals the call on x[b] alone, bit for bit, within a kernel family (up to 8
    tokens: the single-launch kernel; 9 to 64: the streaming kernel); across the two families the partial sums
    are grouped differently, so rows agree to one unit in the last place of the fp16 result.  Repeated calls
    are identical."""
    rng = np.random.default_rng(77)
    m, n = 256, 1024
    p1, p2, su, sv, wscale, inv, W = _trellis_layer(rng, m, n, 4)
    x = cuda(rng.standard_normal((19, n)).astype(np.float32), torch.float16)
    args = (p1, None, su, sv, wscale, 0.0, m, n)
    yb = _run_trellis(ops, x, *args)
    yb2 = _run_trellis(ops, x, *args)
    assert torch.equal(yb, yb2)
    y12 = _run_trellis(ops, x[:12], *args)                 # streaming family, other token-block count
    assert torch.equal(y12, yb[:12])
    y7 = _run_trellis(ops, x[:7], *args)                   # single-launch family
    for b in (0, 3, 6):
        y1 = _run_trellis(ops, x[b:b + 1], *args)
        assert torch.equal(y1[0], y7[b])
        assert torch.equal(y1, _run_trellis(ops, x[b:b + 1], *args))
    ulp = 2.0 ** -10 * yb.float().abs().max().item()
    assert (y7.float() - yb[:7].float()).abs().max().item() <= ulp


@pytest.mark.parametrize("K,K2", [(4, 0), (2, 0), (4, 2)])
@pytest.mark.parametrize("B", [1, 3, 8])
def test_trellis_single_launch_matches_three_launch_form(ops, K, K2, B, monkeypatch):
    """Up to 8 tokens run as ONE kernel (input transform, decode, output transform by the CTA that completes a
    Hadamard block).  Same oracle tolerance as the three-launch form, which stays selectable, and the two agree
    with each other far inside it."""
    rng = np.random.default_rng(300 + K * 10 + K2 + B)
    m, n = 352, 11008 if B == 1 else 576
    p1, p2, su, sv, wscale, inv, W = _trellis_layer(rng, m, n, K, K2)
    x_t = cuda(rng.standard_normal((B, n)).astype(np.float32), torch.bfloat16)
    ref = O.linear_forward(x_t.float().cpu().numpy(), W, su, sv, wscale)
    outs = {}
    for form in ("1", "0"):
        monkeypatch.setenv("GLQB_FUSED_DECODE", form)
        ops.clear_caches()
        y = _run_trellis(ops, x_t, p1, p2, su, sv, wscale, inv, m, n, out_dtype=torch.float32)
        assert relerr(y.cpu().numpy(), ref) <= TOL, form
        plan = next(iter(ops._PLAN_CACHE.values()))
        # inputs wider than 4096 columns are transformed once by a kernel of their own
        assert plan.launches == ((1 if n <= 4096 else 2) if form == "1" else 3)
        outs[form] = y
    assert relerr(outs["1"].cpu().numpy(), outs["0"].cpu().numpy()) <= 1e-5
    ops.clear_caches()


def test_trellis_shards_in_one_launch(ops):
    """q/k/v-style shards that share their input run as one plan and one launch; every shard's output matches the
    oracle within tolerance and the single-layer call to rounding (the work-unit size, hence the grouping of the
    fp32 partial sums, follows the total work of a call); the call can be captured in a CUDA graph."""
    rng = np.random.default_rng(91)
    n, ms = 2048, [2048, 512, 512]
    sv = signs(rng, n)
    layers = []
    for m in ms:
        p1 = rand_packed(rng, m, n, 4)
        layers.append((p1, signs(rng, m), float(np.float16(rng.uniform(0.5, 1.5) * 0.02)), O.trellis_decode_layer(p1, m, n, 4).astype(np.float32)))
    x_t = cuda(rng.standard_normal((2, n)).astype(np.float32), torch.bfloat16)
    sv_t = cuda(sv)
    dev = [(cuda(su), cuda(p1), None, ws, 0.0, m) for (p1, su, ws, W), m in zip(layers, ms)]
    y = ops.fused_linear_trellis_3inst_shards(x_t, sv_t, dev, out_dtype=torch.float32)
    assert y.shape == (2, sum(ms))
    plan = [p for k, p in ops._PLAN_CACHE.items() if k[0] == "trellis_shards"][0]
    assert plan.launches == 1
    col = 0
    for (p1, su, ws, W), (su_t, p_t, _, _, _, m) in zip(layers, dev):
        ref = O.linear_forward(x_t.float().cpu().numpy(), W, su, sv, ws)
        assert relerr(y[:, col:col + m].cpu().numpy(), ref) <= TOL
        single = ops.fused_linear_trellis_3inst(x_t, sv_t, su_t, p_t, None, None, None, None, ws, n, m, n, m,
                                                out_dtype=torch.float32)
        assert relerr(single.cpu().numpy(), y[:, col:col + m].cpu().numpy()) <= 1e-5
        col += m
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        yg = ops.fused_linear_trellis_3inst_shards(x_t, sv_t, dev, out_dtype=torch.float32)
    for _ in range(3):
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(yg, y)
    ops.clear_caches()


def test_trellis_more_than_64_tokens(ops):
    rng = np.random.default_rng(5)
    m, n = 128, 256
    p1, p2, su, sv, wscale, inv, W = _trellis_layer(rng, m, n, 3)
    x = rng.standard_normal((150, n)).astype(np.float32)
    y = _run_trellis(ops, cuda(x), p1, None, su, sv, wscale, 0.0, m, n)
    ref = O.linear_forward(x, W, su, sv, wscale)
    assert relerr(y.cpu().numpy(), ref) <= TOL


def test_trellis_stage2_contributes_and_zero_scale(ops):
    rng = np.random.default_rng(6)
    m, n = 64, 128
    p1, p2, su, sv, wscale, inv, W = _trellis_layer(rng, m, n, 4, 2)
    x = cuda(rng.standard_normal((2, n)).astype(np.float32))
    y_two = _run_trellis(ops, x, p1, p2, su, sv, wscale, inv, m, n)
    y_one = _run_trellis(ops, x, p1, None, su, sv, wscale, 0.0, m, n)
    y_zero = _run_trellis(ops, x, p1, p2, su, sv, wscale, 0.0, m, n)
    assert not torch.allclose(y_two, y_one)
    assert torch.allclose(y_zero, y_one, atol=1e-6)


def test_trellis_yrht_then_shard_transform(ops):
    """Two shards stopped before the output transform, then one transform over both."""
    rng = np.random.default_rng(8)
    n = 256
    ms = [64, 96]
    x = cuda(rng.standard_normal((3, n)).astype(np.float32))
    layers = [_trellis_layer(rng, m, n, 4) for m in ms]
    y_rht = torch.zeros(3, sum(ms), dtype=torch.float32, device="cuda")
    col = 0
    su_all = []
    meta = []
    for m, (p1, p2, su, sv, wscale, inv, W) in zip(ms, layers):
        ops.fused_linear_trellis_3inst_yrht(x, cuda(sv), cuda(p1), torch.tensor(O.block_decompose(n)), None,
                                            wscale, n, n, m, y_rht, col)
        off = col
        for bs in O.block_decompose(m):
            meta.append([off, bs, int(np.log2(bs)), 0])
            off += bs
        col += m
        su_all.append(su)
    y = torch.empty(3, sum(ms), dtype=torch.float32, device="cuda")
    ops.output_rht_shards(y_rht, cuda(np.concatenate(su_all)), y, sum(ms), torch.tensor(meta, dtype=torch.int32), 64)
    col = 0
    for m, (p1, p2, su, sv, wscale, inv, W) in zip(ms, layers):
        ref = O.linear_forward(x.cpu().numpy(), W, su, sv, wscale)
        assert relerr(y[:, col:col + m].cpu().numpy(), ref) <= TOL
        col += m


# ---------------------------------------------------------------------------------------------
# E8 linears
# ---------------------------------------------------------------------------------------------
E8_CASES = ["pow2_1s", "pow2_2s_small", "bd_1s", "bd_2s_full", "bd_3s", "bd_4s"]
_E8_TABLE = {}


def _e8_rot_weight_np(g, name):
    import os
    if "t" not in _E8_TABLE:
        root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
        _E8_TABLE["t"] = O.e8_unpack_table(np.load(os.path.join(root, "glq_b200", "data", "e8_shell_packed.npy")))
    tab = _E8_TABLE["t"]
    fin, fout, m_pad, n_pad, stages, bd, small = [int(v) for v in g[name + "_meta"]]
    qs = [g[f"{name}_Qidxs"], g[f"{name}_Qidxs2"], g[f"{name}_Qidxs3"], g[f"{name}_Qidxs4"]][:stages]
    tabs = [tab, tab[:256] if small else tab, tab, tab][:stages]
    inv = [float(g[f"{name}_inv_resid_scale"]), float(g[f"{name}_inv_resid_scale2"]),
           float(g[f"{name}_inv_resid_scale3"])][:stages - 1]
    return O.e8_decode_nstage(qs, tabs, inv), (fin, fout)


def _e8_args(g, name, e8_cb):
    full, small = e8_cb
    fin, fout, m_pad, n_pad, stages, bd, small_n = [int(v) for v in g[name + "_meta"]]
    empty_i = torch.empty(0, dtype=torch.int16, device="cuda")
    empty_h = torch.empty(0, dtype=torch.float16, device="cuda")
    q = [cuda(g[f"{name}_Qidxs"]), cuda(g[f"{name}_Qidxs2"]), cuda(g[f"{name}_Qidxs3"]), cuda(g[f"{name}_Qidxs4"])]
    inv = [float(g[f"{name}_inv_resid_scale"]), float(g[f"{name}_inv_resid_scale2"]), float(g[f"{name}_inv_resid_scale3"])]
    cb2 = small if small_n else full
    tail = (q[1] if stages >= 2 else empty_i, cb2 if stages >= 2 else empty_h, inv[0] if stages >= 2 else 0.0,
            q[2] if stages >= 3 else empty_i, full if stages >= 3 else empty_h, inv[1] if stages >= 3 else 0.0,
            q[3] if stages >= 4 else empty_i, full if stages >= 4 else empty_h, inv[2] if stages >= 4 else 0.0)
    return fin, fout, m_pad, n_pad, bd, q[0], full, tail


@pytest.mark.parametrize("name", E8_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
def test_e8_linear_vs_reference_golden(ops, golden, e8_cb, name, dtype):
    g = golden("golden_e8_linear.npz")
    fin, fout, m_pad, n_pad, bd, q1, full, tail = _e8_args(g, name, e8_cb)
    x = cuda(g[name + "_x"], dtype)
    su, sv, ws = cuda(g[name + "_SU"]), cuda(g[name + "_SV"]), float(g[name + "_Wscale"])
    if bd:
        y = ops.fused_linear_block_diag(x, sv, su, q1, full, ws, fin, fout, n_pad, m_pad,
                                        torch.tensor(g[name + "_blocks_n"]), torch.tensor(g[name + "_blocks_m"]),
                                        None, None, *tail)
    else:
        y = ops.fused_linear(x, sv, su, q1, full, ws, fin, fout, n_pad, m_pad,
                             int(np.log2(n_pad)), int(np.log2(m_pad)), *tail)
    assert y.shape == (5, fout) and y.dtype == dtype
    # the golden output was computed from fp32 activations; feed the oracle the rounded ones
    W, _ = _e8_rot_weight_np(g, name)
    ref = O.linear_forward(x.float().cpu().numpy(), W, g[name + "_SU"], g[name + "_SV"], ws,
                           list(g[name + "_blocks_n"]), list(g[name + "_blocks_m"]), fout)
    if dtype == torch.float32:
        assert relerr(y.cpu().numpy(), g[name + "_y"]) <= TOL        # against the reference itself
    assert relerr(y.float().cpu().numpy(), ref) <= TOL + OUT_ROUND[dtype]


@pytest.mark.parametrize("stages", [1, 2])
@pytest.mark.parametrize("B", [1, 16, 40])
def test_e8_linear_vs_oracle(ops, e8_table, e8_cb, stages, B):
    """in=out=2048 2 bpw (the reference's CPU-runnable configuration) and the two-stage form."""
    full, small = e8_cb
    rng = np.random.default_rng(stages * 10 + B)
    m = n = 2048
    qs = [rng.integers(0, 65536, size=(m, n // 8), dtype=np.uint16).view(np.int16) for _ in range(stages)]
    inv = [0.1][:stages - 1]
    su, sv = signs(rng, m), signs(rng, n)
    wscale = float(rng.uniform(0.5, 1.5) * 0.02)
    W = O.e8_decode_nstage(qs, [e8_table] * stages, inv)
    x = cuda(rng.standard_normal((B, n)).astype(np.float32), torch.bfloat16)
    empty_i = torch.empty(0, dtype=torch.int16, device="cuda")
    empty_h = torch.empty(0, dtype=torch.float16, device="cuda")
    y = ops.fused_linear(x, cuda(sv), cuda(su), cuda(qs[0]), full, wscale, n, m, n, m, 11, 11,
                         cuda(qs[1]) if stages > 1 else empty_i, full if stages > 1 else empty_h,
                         inv[0] if stages > 1 else 0.0, out_dtype=torch.float32)
    ref = O.linear_forward(x.float().cpu().numpy(), W, su, sv, wscale)
    assert relerr(y.cpu().numpy(), ref) <= TOL
    y2 = ops.fused_linear(x, cuda(sv), cuda(su), cuda(qs[0]), full, wscale, n, m, n, m, 11, 11,
                          cuda(qs[1]) if stages > 1 else empty_i, full if stages > 1 else empty_h,
                          inv[0] if stages > 1 else 0.0, out_dtype=torch.float32)
    assert torch.equal(y, y2)


def test_e8_per_row_scale_superset(e8_table, e8_cb):
    """Per-row scale (used only by the synthetic benchmark configuration) through the plan API."""
    from glq_b200 import _lib
    from glq_b200.ops import e8_packed_table
    from glq_b200.plan import LinearSpec, Plan
    full, _ = e8_cb
    rng = np.random.default_rng(42)
    m = n = 512
    q = rng.integers(0, 65536, size=(m, n // 8), dtype=np.uint16).view(np.int16)
    su, sv = signs(rng, m), signs(rng, n)
    rs = (rng.uniform(0.5, 1.5, size=m) * 0.02).astype(np.float32)
    x = cuda(rng.standard_normal((2, n)).astype(np.float32))
    y = torch.empty(2, m, dtype=torch.float32, device="cuda")
    spec = LinearSpec(format=_lib.FMT_E8_SHELL, m_pad=m, n_pad=n, in_features=n, out_features=m, codes=[cuda(q)],
                      tables=[e8_packed_table(full)], su=cuda(su), sv=cuda(sv), wscale=1.0, row_scale=cuda(rs),
                      batch=2, x_dtype=torch.float32, y_dtype=torch.float32)
    Plan([spec]).run(x, y)
    ref = O.linear_forward(x.cpu().numpy(), O.e8_decode(q, e8_table), su, sv, 1.0, row_scale=rs)
    assert relerr(y.cpu().numpy(), ref) <= TOL


def test_e8_unfused_pieces(ops, e8_table, e8_cb):
    """input_rht -> dequant_matmul -> output_rht equals the fused op."""
    full, _ = e8_cb
    rng = np.random.default_rng(11)
    m, n, fin, fout = 128, 256, 200, 100
    q = rng.integers(0, 65536, size=(m, n // 8), dtype=np.uint16).view(np.int16)
    su, sv = signs(rng, m), signs(rng, n)
    x = cuda(rng.standard_normal((4, fin)).astype(np.float32))
    x_rht = torch.empty(4, n, dtype=torch.float32, device="cuda")
    ops.input_rht(x, cuda(sv), x_rht, fin, fin, 1 / 16.0, n, 8)
    xr_ref = O.block_diag_fht(np.pad(x.cpu().numpy(), ((0, 0), (0, n - fin))) * sv.astype(np.float32), [n])
    np.testing.assert_allclose(x_rht.cpu().numpy(), xr_ref, atol=1e-5)
    y_rht = ops.dequant_matmul(x_rht, cuda(q), full, 0.03)
    W = O.e8_decode(q, e8_table)
    assert relerr(y_rht.cpu().numpy(), xr_ref @ W.T * 0.03) <= TOL
    y = torch.empty(4, fout, dtype=torch.float32, device="cuda")
    ops.output_rht(y_rht, cuda(su), y, fout, m, 7, 1 / np.sqrt(m))
    ref = O.linear_forward(x.cpu().numpy(), W, su, sv, 0.03, [n], [m], fout)
    assert relerr(y.cpu().numpy(), ref) <= TOL


def test_shared_input_plan_matches_single_layers(ops):
    """q/k/v-style plan: three layers sharing one input and one output tensor."""
    from glq_b200 import _lib
    from glq_b200.plan import LinearSpec, Plan
    rng = np.random.default_rng(21)
    n, ms = 512, [256, 64, 64]
    x = cuda(rng.standard_normal((1, n)).astype(np.float32), torch.bfloat16)
    sv = cuda(signs(rng, n))
    layers = [_trellis_layer(rng, m, n, 4) for m in ms]
    y = torch.zeros(1, sum(ms), dtype=torch.bfloat16, device="cuda")
    specs, off, keep = [], 0, []
    for m, (p1, p2, su, _sv, wscale, inv, W) in zip(ms, layers):
        specs.append(LinearSpec(format=_lib.FMT_TRELLIS_3INST, m_pad=m, n_pad=n, in_features=n, out_features=m,
                                codes=[cuda(p1)], bits=[4], su=cuda(su), sv=sv, wscale=wscale, batch=1,
                                y_stride=sum(ms), y_offset=off))
        off += m
    plan = Plan(specs)
    plan.run(x, y)
    off = 0
    for m, (p1, p2, su, _sv, wscale, inv, W) in zip(ms, layers):
        ref = O.linear_forward(x.float().cpu().numpy(), W, su, sv.cpu().numpy(), wscale)
        assert relerr(y[:, off:off + m].float().cpu().numpy(), ref) <= TOL + OUT_ROUND[torch.bfloat16]
        off += m


def test_errors_are_loud(ops):
    with pytest.raises(RuntimeError):
        ops.glq_decompress_trellis_3inst_cuda(torch.zeros(4, 64, dtype=torch.int16, device="cuda"), 48, 64)
    with pytest.raises(RuntimeError):
        ops.glq_decompress_trellis_3inst_cuda(torch.zeros(4, 64, dtype=torch.int16), 32, 32)   # CPU tensor


# ---------------------------------------------------------------------------------------------
# prefill: tensor-core GEMM path (more than 64 tokens)
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("K,K2", [(4, 0), (2, 0), (3, 0), (4, 2)])
@pytest.mark.parametrize("T", [65, 128, 200, 300])
def test_trellis_gemm_vs_oracle(ops, K, K2, T):
    rng = np.random.default_rng(K * 1000 + K2 * 100 + T)
    m, n = 352, 576            # partial 128-row tile, 9 K chunks, block-diagonal transforms
    p1, p2, su, sv, wscale, inv, W = _trellis_layer(rng, m, n, K, K2)
    x_t = cuda(rng.standard_normal((T, n)).astype(np.float32), torch.bfloat16)
    ref = O.linear_forward(x_t.float().cpu().numpy(), W, su, sv, wscale)
    y = _run_trellis(ops, x_t, p1, p2, su, sv, wscale, inv, m, n, out_dtype=torch.float32)
    assert y.shape == (T, m)
    assert relerr(y.cpu().numpy(), ref) <= TOL
    y2 = _run_trellis(ops, x_t, p1, p2, su, sv, wscale, inv, m, n, out_dtype=torch.float32)
    assert torch.equal(y, y2)


def test_trellis_gemm_large(ops):
    rng = np.random.default_rng(31)
    m, n, T = 2048, 2048, 512
    p1, p2, su, sv, wscale, inv, W = _trellis_layer(rng, m, n, 4)
    x_t = cuda(rng.standard_normal((T, n)).astype(np.float32), torch.bfloat16)
    ref = O.linear_forward(x_t.float().cpu().numpy(), W, su, sv, wscale)
    y = _run_trellis(ops, x_t, p1, None, su, sv, wscale, 0.0, m, n, out_dtype=torch.float32)
    assert relerr(y.cpu().numpy(), ref) <= TOL
    # rows of the GEMM result agree with the decode path on the same tokens (not bit-equal: the
    # accumulation order differs)
    y1 = _run_trellis(ops, x_t[:5], p1, None, su, sv, wscale, 0.0, m, n, out_dtype=torch.float32)
    assert relerr(y[:5].cpu().numpy(), y1.cpu().numpy()) <= 1e-4


@pytest.mark.parametrize("stages", [1, 2, 4])
@pytest.mark.parametrize("T", [100, 257, 600])       # 600 tokens: weight tiles decoded once, then a bulk-copy-fed GEMM
def test_e8_gemm_vs_oracle(ops, e8_table, e8_cb, stages, T):
    full, small = e8_cb
    rng = np.random.default_rng(stages * 7 + T)
    m, n = 320, 576
    qs = [rng.integers(0, 65536, size=(m, n // 8), dtype=np.uint16).view(np.int16) for _ in range(stages)]
    inv = [0.1, 0.01, 0.001][:stages - 1]
    su, sv = signs(rng, m), signs(rng, n)
    wscale = float(rng.uniform(0.5, 1.5) * 0.02)
    W = O.e8_decode_nstage(qs, [e8_table] * stages, inv)
    x = cuda(rng.standard_normal((T, n)).astype(np.float32), torch.bfloat16)
    empty_i = torch.empty(0, dtype=torch.int16, device="cuda")
    empty_h = torch.empty(0, dtype=torch.float16, device="cuda")
    tail = []
    for s in range(1, 4):
        tail += [cuda(qs[s]) if stages > s else empty_i, full if stages > s else empty_h, inv[s - 1] if stages > s else 0.0]
    y = ops.fused_linear_block_diag(x, cuda(sv), cuda(su), cuda(qs[0]), full, wscale, n, m, n, m,
                                    torch.tensor(O.block_decompose(n)), torch.tensor(O.block_decompose(m)), None, None,
                                    *tail, out_dtype=torch.float32)
    ref = O.linear_forward(x.float().cpu().numpy(), W, su, sv, wscale)
    assert relerr(y.cpu().numpy(), ref) <= TOL


# ---------------------------------------------------------------------------------------------
# E8 decode with most of the codebook resident in the shared memory of one CTA per SM
# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("stages,small2", [(1, False), (2, False), (2, True), (4, False)])
@pytest.mark.parametrize("B", [1, 9])
def test_e8_resident_table_path_matches_oracle_and_global_path(ops, e8_table, e8_cb, monkeypatch, stages, small2, B):
    full, small = e8_cb
    rng = np.random.default_rng(stages * 31 + B + int(small2))
    m, n = 320, 832
    qs = [rng.integers(0, 65536, size=(m, n // 8), dtype=np.uint16).view(np.int16) for _ in range(stages)]
    tabs = [e8_table] * stages
    if small2:
        qs[1] = rng.integers(0, 256, size=(m, n // 8), dtype=np.uint16).view(np.int16)
        tabs[1] = e8_table[:256]
    inv = [0.3, 0.09, 0.027][:stages - 1]
    su, sv = signs(rng, m), signs(rng, n)
    W = O.e8_decode_nstage(qs, tabs, inv)
    x = cuda(rng.standard_normal((B, n)).astype(np.float32), torch.float16)
    empty_i = torch.empty(0, dtype=torch.int16, device="cuda")
    empty_h = torch.empty(0, dtype=torch.float16, device="cuda")
    tail = []
    for s in range(1, 4):
        cb = small if (s == 1 and small2) else full
        tail += [cuda(qs[s]) if stages > s else empty_i, cb if stages > s else empty_h, inv[s - 1] if stages > s else 0.0]
    args = (x, cuda(sv), cuda(su), cuda(qs[0]), full, 0.02, n, m, n, m,
            torch.tensor(O.block_decompose(n)), torch.tensor(O.block_decompose(m)), None, None, *tail)
    ops.clear_caches()
    monkeypatch.setenv("GLQB_FUSED_DECODE", "0")               # the streaming kernels (not the single-launch form)
    monkeypatch.setenv("GLQB_E8_SMEM_MIN_BYTES", "0")          # force the shared-memory table path
    y_smem = ops.fused_linear_block_diag(*args, out_dtype=torch.float32)
    ops.clear_caches()
    monkeypatch.setenv("GLQB_E8_SMEM_MIN_BYTES", str(1 << 40))  # force the global-memory gathers
    y_glob = ops.fused_linear_block_diag(*args, out_dtype=torch.float32)
    ops.clear_caches()
    ref = O.linear_forward(x.float().cpu().numpy(), W, su, sv, 0.02)
    assert relerr(y_smem.cpu().numpy(), ref) <= TOL
    assert relerr(y_smem.cpu().numpy(), y_glob.cpu().numpy()) <= 1e-5


@pytest.mark.parametrize("stages,small2", [(1, False), (2, False), (2, True), (3, False), (4, False)])
@pytest.mark.parametrize("B", [1, 3, 8])
def test_e8_single_launch_matches_three_launch_form(ops, e8_table, e8_cb, monkeypatch, stages, small2, B):
    """Up to 8 tokens an E8 layer runs as ONE kernel too (input transform, gathers + matvec, output transform by the
    CTA that completes a Hadamard block); the three-launch form stays selectable and the two agree far inside the
    oracle tolerance.  A batch-1 case is wide enough (5376 columns) to have its input transformed by a kernel of
    its own; n = 832 leaves a ragged last column group; m = 328 has an 8-row Hadamard block, shorter than a strip,
    and must keep the three-launch form."""
    full, small = e8_cb
    rng = np.random.default_rng(900 + stages * 31 + B + int(small2))
    m, n = (5376, 5376) if (B == 1 and stages == 2 and not small2) else (328 if B == 3 else 320, 832)
    qs = [rng.integers(0, 65536, size=(m, n // 8), dtype=np.uint16).view(np.int16) for _ in range(stages)]
    tabs = [e8_table] * stages
    if small2:
        qs[1] = rng.integers(0, 256, size=(m, n // 8), dtype=np.uint16).view(np.int16)
        tabs[1] = e8_table[:256]
    inv = [0.3, 0.09, 0.027][:stages - 1]
    su, sv = signs(rng, m), signs(rng, n)
    W = O.e8_decode_nstage(qs, tabs, inv)
    x = cuda(rng.standard_normal((B, n)).astype(np.float32), torch.bfloat16)
    empty_i = torch.empty(0, dtype=torch.int16, device="cuda")
    empty_h = torch.empty(0, dtype=torch.float16, device="cuda")
    tail = []
    for s in range(1, 4):
        cb = small if (s == 1 and small2) else full
        tail += [cuda(qs[s]) if stages > s else empty_i, cb if stages > s else empty_h, inv[s - 1] if stages > s else 0.0]
    args = (x, cuda(sv), cuda(su), cuda(qs[0]), full, 0.02, n, m, n, m,
            torch.tensor(O.block_decompose(n)), torch.tensor(O.block_decompose(m)), None, None, *tail)
    ref = O.linear_forward(x.float().cpu().numpy(), W, su, sv, 0.02)
    outs = {}
    # "1": gathers through L1 / L2 (small launches); "res": most of the codebook copied into shared memory first (what
    # launches of a few MB do by themselves); "0": three launches
    for form in ("1", "res", "0"):
        monkeypatch.setenv("GLQB_FUSED_DECODE", "0" if form == "0" else "1")
        monkeypatch.setenv("GLQB_E8_FUSED_RES_MIN_BYTES", "0" if form == "res" else str(1 << 40))
        ops.clear_caches()
        y = ops.fused_linear_block_diag(*args, out_dtype=torch.float32)
        assert relerr(y.cpu().numpy(), ref) <= TOL, form
        plan = next(iter(ops._PLAN_CACHE.values()))
        # 328 rows decompose into 256 + 64 + 8: a block shorter than a 16-row strip keeps the three-launch form
        single = (1 if n <= 4096 else 2) if m != 328 else 3
        assert plan.launches == (single if form != "0" else 3), (form, plan.launches)
        outs[form] = y
    assert relerr(outs["1"].cpu().numpy(), outs["0"].cpu().numpy()) <= 1e-5
    assert torch.equal(outs["1"], outs["res"])               # same arithmetic, only the source of the table entries differs
    ops.clear_caches()


def test_glq_linear_module_matches_oracle(e8_table, e8_cb):
    """The E8RHTLinear mirror: load reference-named buffers, forward on the GPU, compare with the oracle."""
    from glq_b200.linear import GLQLinear
    full, small = e8_cb
    rng = np.random.default_rng(12)
    lin = GLQLinear(200, 100, bias=True)                       # power-of-two padded: 256 x 128
    q1 = rng.integers(0, 65536, size=(128, 32), dtype=np.uint16).view(np.int16)
    q2 = rng.integers(0, 256, size=(128, 32), dtype=np.uint16).view(np.int16)
    su, sv = signs(rng, 128), signs(rng, 256)
    sd = {"Qidxs": torch.from_numpy(q1.copy()), "Qidxs2": torch.from_numpy(q2.copy()), "SU": torch.from_numpy(su),
          "SV": torch.from_numpy(sv), "Wscale": torch.tensor(0.04), "inv_resid_scale": torch.tensor(0.3),
          "bias": torch.from_numpy(rng.standard_normal(100).astype(np.float16))}
    lin.load_state_dict(sd, strict=False)
    lin = lin.cuda()
    lin.set_codebook(full, codebook2=small)
    x = cuda(rng.standard_normal((2, 3, 200)).astype(np.float32))
    y = lin(x)
    assert y.shape == (2, 3, 100)
    W = O.e8_decode_nstage([q1, q2], [e8_table, e8_table[:256]], [np.float32(0.3)])
    ref = O.linear_forward(x.cpu().numpy().reshape(6, 200), W, su, sv, 0.04, [256], [128], 100) + sd["bias"].float().numpy()
    assert relerr(y.cpu().numpy().reshape(6, 100), ref) <= TOL
    assert np.array_equal(lin.dequantize_rotated().cpu().numpy().view(np.uint32), W.view(np.uint32))

    tl = GLQLinear(576, 352, codebook_type="trellis")
    p1 = rand_packed(rng, 352, 576, 4)
    tsu, tsv = signs(rng, 352), signs(rng, 576)
    tl.load_state_dict({"trellis_packed": torch.from_numpy(p1.copy()), "SU": torch.from_numpy(tsu),
                        "SV": torch.from_numpy(tsv), "Wscale": torch.tensor(0.02)}, strict=False)
    tl = tl.cuda()
    xt = cuda(rng.standard_normal((4, 576)).astype(np.float32))
    Wt = O.trellis_decode_layer(p1, 352, 576, 4).astype(np.float32)
    assert relerr(tl(xt).cpu().numpy(), O.linear_forward(xt.cpu().numpy(), Wt, tsu, tsv, 0.02)) <= TOL


# ---------------------------------------------------------------------------------------------
# edge cases: empty and ragged inputs, strided rows
# ---------------------------------------------------------------------------------------------
def test_empty_batch_returns_empty(ops):
    rng = np.random.default_rng(77)
    m, n = 64, 128
    p1, p2, su, sv, wscale, inv, W = _trellis_layer(rng, m, n, 4)
    x_t = torch.zeros(0, n, dtype=torch.bfloat16, device="cuda")
    y = _run_trellis(ops, x_t, p1, None, su, sv, wscale, 0.0, m, n)
    assert y.shape == (0, m) and y.dtype == torch.bfloat16


def test_leading_dims_and_strided_rows(ops):
    """(2, 3, n) activations are flattened like the reference does (x.reshape(-1, in_features)); rows that are
    a strided view (every second row of a larger buffer) are read in place, without a copy."""
    rng = np.random.default_rng(78)
    m, n = 96, 192
    p1, p2, su, sv, wscale, inv, W = _trellis_layer(rng, m, n, 3)
    x = rng.standard_normal((2, 3, n)).astype(np.float32)
    x_t = cuda(x, torch.float16)
    ref = O.linear_forward(x_t.float().cpu().numpy().reshape(-1, n), W, su, sv, wscale)
    y = _run_trellis(ops, x_t, p1, None, su, sv, wscale, 0.0, m, n, out_dtype=torch.float32)
    assert y.shape == (6, m)
    assert relerr(y.cpu().numpy(), ref) <= TOL
    big = torch.zeros(12, n, dtype=torch.float16, device="cuda")
    big[::2] = x_t.reshape(6, n)
    ys = _run_trellis(ops, big[::2], p1, None, su, sv, wscale, 0.0, m, n, out_dtype=torch.float32)
    assert torch.equal(ys, y)


@pytest.mark.parametrize("T", [1, 9, 33, 64])
def test_ragged_token_counts_match_row_by_row(ops, T, monkeypatch):
    """Token counts that do not fill the 8-token MMA column blocks: every row equals the batch-1 result of the
    same kernel family bit for bit (the streaming kernels here: the single-launch form is switched off)."""
    rng = np.random.default_rng(500 + T)
    m, n = 64, 256
    p1, p2, su, sv, wscale, inv, W = _trellis_layer(rng, m, n, 4)
    x_t = cuda(rng.standard_normal((T, n)).astype(np.float32), torch.bfloat16)
    monkeypatch.setenv("GLQB_FUSED_DECODE", "0")
    ops.clear_caches()
    y = _run_trellis(ops, x_t, p1, None, su, sv, wscale, 0.0, m, n, out_dtype=torch.float32)
    for r in (0, T // 2, T - 1):
        y1 = _run_trellis(ops, x_t[r:r + 1], p1, None, su, sv, wscale, 0.0, m, n, out_dtype=torch.float32)
        assert torch.equal(y[r:r + 1], y1)
    ops.clear_caches()


@pytest.mark.parametrize("stages,small2", [(1, False), (2, False), (2, True), (3, False)])
def test_e8_two_phase_prefill_resident_table_equals_global_table(ops, e8_table, e8_cb, monkeypatch, stages, small2):
    """More than 256 tokens: weight tiles are decoded once, with the codebook either gathered from global memory
    or resident in shared memory.  Both forms must produce the same tiles, hence bit-equal outputs."""
    full, small = e8_cb
    rng = np.random.default_rng(900 + stages * 7 + int(small2))
    m, n, T = 320, 832, 300
    qs = [rng.integers(0, 65536, size=(m, n // 8), dtype=np.uint16).view(np.int16) for _ in range(stages)]
    tabs = [e8_table] * stages
    if small2:
        qs[1] = rng.integers(0, 256, size=(m, n // 8), dtype=np.uint16).view(np.int16)
        tabs[1] = e8_table[:256]
    inv = [0.3, 0.09, 0.027][:stages - 1]
    su, sv = signs(rng, m), signs(rng, n)
    W = O.e8_decode_nstage(qs, tabs, inv)
    x = cuda(rng.standard_normal((T, n)).astype(np.float32), torch.float16)
    empty_i = torch.empty(0, dtype=torch.int16, device="cuda")
    empty_h = torch.empty(0, dtype=torch.float16, device="cuda")
    tail = []
    for s in range(1, 4):
        cb = small if (s == 1 and small2) else full
        tail += [cuda(qs[s]) if stages > s else empty_i, cb if stages > s else empty_h, inv[s - 1] if stages > s else 0.0]
    args = (x, cuda(sv), cuda(su), cuda(qs[0]), full, 0.02, n, m, n, m,
            torch.tensor(O.block_decompose(n)), torch.tensor(O.block_decompose(m)), None, None, *tail)
    ops.clear_caches()
    monkeypatch.setenv("GLQB_E8_SMEM_MIN_BYTES", "0")
    y_smem = ops.fused_linear_block_diag(*args, out_dtype=torch.float32)
    ops.clear_caches()
    monkeypatch.setenv("GLQB_E8_SMEM_MIN_BYTES", str(1 << 40))
    y_glob = ops.fused_linear_block_diag(*args, out_dtype=torch.float32)
    ops.clear_caches()
    ref = O.linear_forward(x.float().cpu().numpy(), W, su, sv, 0.02)
    assert relerr(y_glob.cpu().numpy(), ref) <= TOL
    assert torch.equal(y_smem, y_glob)
