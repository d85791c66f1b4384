"""GPU parity at the sizes the benchmark figures are quoted on, each against the CPU oracle through the C ABI:

* Llama-3-8B shaped E8 two-stage layers (14336 x 4096, 4096 x 14336): prefill GEMM at 2048 tokens (every
  row compared), the streaming kernels at 1 and 16 tokens with the table in global and in shared memory;
* the 62-layer shapes (21504 x 5376, 5376 x 21504, three stages, Hadamard block 16384) at 1 and 256 tokens;
* the MoE step of 128 experts, top-8, hidden 2048, expert intermediate 768: 256 tokens with near-uniform and
  Zipf(1.2) routing, 4096 tokens (tensor-core form) on a sample of 64 tokens;
* E8-shell experts (grouped / block-diagonal MoE ops), activation codes 3-5, the two-stage "_yrht" op, the
  stateless C entry point, unaligned index rows, plan bucketing, dequantize(), shared-memory limits.

Tolerance: max|y - ref| / max|ref| <= 2e-3 on fp32 results (plus half an ulp of the output type for 16-bit
results); MoE 5e-3 (two chained layers with fp16 hand-offs; the reference's own gate is rtol = atol = 2e-2).
"""
import ctypes as C
import os

import numpy as np
import pytest
import torch

from oracle import c_oracle as CO
from oracle import glq_oracle as O

pytestmark = pytest.mark.gpu

TOL = 2e-3
MOE_TOL = 5e-3
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def relerr(y, ref):
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    return np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30)


def cuda(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def signs(rng, *shape):
    return (rng.integers(0, 2, size=shape) * 2 - 1).astype(np.float16)


def idx(rng, *shape):
    return rng.integers(0, 65536, size=shape, dtype=np.uint16).view(np.int16)


@pytest.fixture(scope="module")
def ops():
    from glq_b200 import ops as _ops
    yield _ops
    _ops.clear_caches()


@pytest.fixture(scope="module")
def packed_table():
    return np.load(os.path.join(ROOT, "glq_b200", "data", "e8_shell_packed.npy"))


@pytest.fixture(scope="module")
def cb16(packed_table):
    return cuda(O.e8_unpack_table(packed_table).astype(np.float16))


def _e8_layer(rng, m, n, stages, packed_table, inv0=0.1):
    qs = [idx(rng, m, n // 8) for _ in range(stages)]
    inv = [inv0 ** (s + 1) for s in range(stages - 1)]
    W = CO.e8_decode(qs, [packed_table] * stages, inv, m, n)
    return qs, inv, W, signs(rng, m), signs(rng, n), float(np.float16(rng.uniform(0.5, 1.5) * 0.02))


def _run_e8(ops, x_t, qs, inv, su, sv, ws, m, n, cb, out_dtype=torch.float32):
    ei = torch.empty(0, dtype=torch.int16, device="cuda")
    eh = torch.empty(0, dtype=torch.float16, device="cuda")
    tail = []
    for s in range(1, 4):
        tail += [cuda(qs[s]), cb, inv[s - 1]] if s < len(qs) else [ei, eh, 0.0]
    return ops.fused_linear_block_diag(x_t, cuda(sv), cuda(su), cuda(qs[0]), cb, ws, n, m, n, m,
                                       torch.tensor(O.block_decompose(n)), torch.tensor(O.block_decompose(m)),
                                       None, None, *tail, out_dtype=out_dtype)


# ---------------------------------------------------------------------------------------------------------
# Llama-3-8B shapes, E8 two-stage (4 bpw)
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(14336, 4096), (4096, 14336)])
def test_e8_two_stage_llama_shapes(ops, packed_table, cb16, shape, monkeypatch):
    m, n = shape
    rng = np.random.default_rng(m * 3 + n)
    qs, inv, W, su, sv, ws = _e8_layer(rng, m, n, 2, packed_table)
    dump = ops.dequant_e8([cuda(q) for q in qs], [cb16, cb16], inv).cpu().numpy()
    assert np.array_equal(dump.view(np.uint32), W.view(np.uint32))            # reconstructed weights: bit exact
    # prefill, 2048 tokens, tensor-core path, every row
    x = rng.standard_normal((2048, n)).astype(np.float32)
    x_t = cuda(x, torch.bfloat16)
    xf = x_t.float().cpu().numpy()
    ref = O.linear_forward(xf, W, su, sv, ws)
    y = _run_e8(ops, x_t, qs, inv, su, sv, ws, m, n, cb16)
    assert relerr(y.cpu().numpy(), ref) <= TOL
    y2 = _run_e8(ops, x_t, qs, inv, su, sv, ws, m, n, cb16)
    assert torch.equal(y, y2)
    # the GEMM folds both stages into one fp16 operand, fp16(w1 + fp16(s) * w2), one rounding: the result must
    # be closer still to a reference built from exactly those operands
    s16 = np.float32(np.float16(inv[0]))
    w1 = CO.e8_decode(qs[:1], [packed_table], [], m, n)
    w2 = CO.e8_decode(qs[1:], [packed_table], [], m, n)
    Wf = (w1.astype(np.float64) + np.float64(s16) * w2.astype(np.float64)).astype(np.float16).astype(np.float32)
    assert np.abs(Wf - W).max() <= 2.0 ** -11 * np.abs(W).max() * 1.01         # half an fp16 ulp of the largest weight
    assert relerr(y.cpu().numpy(), O.linear_forward(xf, Wf, su, sv, ws)) <= TOL / 2
    # decode: 1 and 16 tokens, table gathered from global memory and resident in shared memory
    for min_bytes in ("1000000000000", "0"):
        monkeypatch.setenv("GLQB_E8_SMEM_MIN_BYTES", min_bytes)
        ops.clear_caches()
        for T in (1, 16):
            yt = _run_e8(ops, x_t[:T], qs, inv, su, sv, ws, m, n, cb16)
            assert relerr(yt.cpu().numpy(), ref[:T]) <= TOL, (min_bytes, T)
            assert torch.equal(yt, _run_e8(ops, x_t[:T], qs, inv, su, sv, ws, m, n, cb16))
    ops.clear_caches()


# ---------------------------------------------------------------------------------------------------------
# 62-layer dense decoder shapes: three E8 stages, Hadamard blocks 16384 + 4096 + 1024
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(21504, 5376), (5376, 21504)])
def test_e8_three_stage_dense62_shapes(ops, packed_table, cb16, shape):
    m, n = shape
    rng = np.random.default_rng(m + 7 * n)
    qs, inv, W, su, sv, ws = _e8_layer(rng, m, n, 3, packed_table)
    x = rng.standard_normal((256, n)).astype(np.float32)
    x_t = cuda(x, torch.bfloat16)
    ref = O.linear_forward(x_t.float().cpu().numpy(), W, su, sv, ws)
    y1 = _run_e8(ops, x_t[:1], qs, inv, su, sv, ws, m, n, cb16)
    assert relerr(y1.cpu().numpy(), ref[:1]) <= TOL
    y = _run_e8(ops, x_t, qs, inv, su, sv, ws, m, n, cb16)
    assert relerr(y.cpu().numpy(), ref) <= TOL
    yb = _run_e8(ops, x_t, qs, inv, su, sv, ws, m, n, cb16, out_dtype=torch.bfloat16)
    assert torch.equal(yb, y.to(torch.bfloat16))
    ops.clear_caches()


def test_trellis_prefill_2048_tokens_smollm_gate(ops):
    """SmolLM3-3B gate projection (11008 x 2048, 4 bpw) at 2048 tokens: the trellis tensor-core path."""
    m, n = 11008, 2048
    rng = np.random.default_rng(11)
    packed = idx(rng, (m // 16) * (n // 16), 64)
    W = CO.trellis_decode(packed, m, n, 4).astype(np.float32)
    su, sv, ws = signs(rng, m), signs(rng, n), 0.017
    x_t = cuda(rng.standard_normal((2048, n)).astype(np.float32), torch.bfloat16)
    ref = O.linear_forward(x_t.float().cpu().numpy(), W, su, sv, ws)
    y = ops.fused_linear_trellis_3inst(x_t, cuda(sv), cuda(su), cuda(packed), None, None, None, None, ws, n, m, n, m,
                                       out_dtype=torch.float32)
    assert relerr(y.cpu().numpy(), ref) <= TOL
    ops.clear_caches()


# ---------------------------------------------------------------------------------------------------------
# MoE: 128 experts, top-8, hidden 2048, expert intermediate 768, trellis 4 bpw, gelu-tanh gate
# ---------------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def moe128():
    E, hidden, inter = 128, 2048, 768
    rng = np.random.default_rng(128768)
    w13_out = 2 * inter
    d = dict(w13=idx(rng, E, (w13_out // 16) * (hidden // 16), 64), w2=idx(rng, E, (hidden // 16) * (inter // 16), 64),
             su13=signs(rng, E, w13_out), sv13=signs(rng, hidden), su2=signs(rng, E, hidden), sv2=signs(rng, inter),
             ws13=(rng.uniform(0.5, 1.5, size=E) * 0.02).astype(np.float32),
             ws2=(rng.uniform(0.5, 1.5, size=E) * 0.02).astype(np.float32))
    dev = {k: cuda(v) for k, v in d.items()}
    cache = {}

    def weights(e):
        if e not in cache:
            cache[e] = (CO.trellis_decode(d["w13"][e], w13_out, hidden, 4).astype(np.float32),
                        CO.trellis_decode(d["w2"][e], hidden, inter, 4).astype(np.float32))
        return cache[e]
    return d, dev, weights, (E, hidden, inter, w13_out)


def _moe128_oracle(moe, x, ids, w):
    d, dev, weights, (E, hidden, inter, w13_out) = moe
    f16 = lambda a: a.astype(np.float16).astype(np.float32)
    f13 = lambda e, xb: f16(O.linear_forward(xb, weights(e)[0], d["su13"][e], d["sv13"], float(d["ws13"][e])))
    f2 = lambda e, hb: f16(O.linear_forward(f16(hb), weights(e)[1], d["su2"][e], d["sv2"], float(d["ws2"][e])))
    return O.moe_forward(x, ids, w, f13, f2, inter, "gelu_tanh")


def _moe128_run(ops, moe, x_t, ids_t, w_t):
    d, dev, weights, (E, hidden, inter, w13_out) = moe
    sentinel = torch.zeros(E, 1, 1, dtype=torch.int16, device="cuda")
    bl = lambda n: torch.tensor(O.block_decompose(n))
    return ops.fused_moe_trellis_3inst(
        x_t, ids_t, w_t, dev["w13"], sentinel, dev["su13"], dev["sv13"], dev["ws13"], dev["ws13"],
        dev["w2"], sentinel, dev["su2"], dev["sv2"], dev["ws2"], dev["ws2"], hidden, inter, w13_out,
        hidden, w13_out, inter, hidden, bl(hidden), bl(w13_out), None, None, bl(inter), bl(hidden), None, None, 1)


def _routing(rng, T, E, k, zipf):
    if zipf:
        p = np.arange(1, E + 1, dtype=np.float64) ** -1.2
        p /= p.sum()
        ids = np.stack([rng.choice(E, size=k, replace=False, p=p) for _ in range(T)]).astype(np.int64)
        w = rng.random((T, k)).astype(np.float32)
    else:
        logits = rng.standard_normal((T, E))
        ids = np.argsort(-logits, axis=1)[:, :k].astype(np.int64)
        ex = np.exp(np.take_along_axis(logits, ids, axis=1))
        w = ex.astype(np.float32)
    return ids, (w / w.sum(1, keepdims=True)).astype(np.float32)


@pytest.mark.parametrize("zipf", [False, True])
def test_moe_128_experts_256_tokens(ops, moe128, zipf):
    E, hidden, inter, w13_out = moe128[3]
    rng = np.random.default_rng(256 + zipf)
    T, k = 256, 8
    ids, w = _routing(rng, T, E, k, zipf)
    x_t = cuda(rng.standard_normal((T, hidden)).astype(np.float32), torch.bfloat16)
    y = _moe128_run(ops, moe128, x_t, cuda(ids), cuda(w))
    assert torch.equal(y, _moe128_run(ops, moe128, x_t, cuda(ids), cuda(w)))
    ref = _moe128_oracle(moe128, x_t.float().cpu().numpy(), ids, w)
    assert relerr(y.float().cpu().numpy(), ref) <= MOE_TOL + 2.0 ** -8


def test_moe_128_experts_4096_tokens_sampled(ops, moe128):
    """256 routed tokens per expert on average: the tensor-core form.  Token outputs are independent of each
    other, so the oracle is evaluated for a sample of 64 tokens only."""
    E, hidden, inter, w13_out = moe128[3]
    rng = np.random.default_rng(4096)
    T, k = 4096, 8
    ids, w = _routing(rng, T, E, k, False)
    x_t = cuda(rng.standard_normal((T, hidden)).astype(np.float32), torch.bfloat16)
    y = _moe128_run(ops, moe128, x_t, cuda(ids), cuda(w))
    sel = np.sort(rng.choice(T, size=64, replace=False))
    ref = _moe128_oracle(moe128, x_t.float().cpu().numpy()[sel], ids[sel], w[sel])
    assert relerr(y.float().cpu().numpy()[sel], ref) <= MOE_TOL + 2.0 ** -8
    ops.clear_caches()


# ---------------------------------------------------------------------------------------------------------
# MoE activation codes without a gate (3 silu, 4 gelu, 5 relu^2): w13 has `inter` rows
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("act", [3, 4, 5])
@pytest.mark.parametrize("T", [5, 300])
def test_moe_plain_activations(ops, act, T):
    E, hidden, inter, k = 8, 256, 128, 2
    rng = np.random.default_rng(900 + act + T)
    w13 = idx(rng, E, (inter // 16) * (hidden // 16), 64)
    w2 = idx(rng, E, (hidden // 16) * (inter // 16), 64)
    su13, sv13, su2, sv2 = signs(rng, E, inter), signs(rng, hidden), signs(rng, E, hidden), signs(rng, inter)
    ws13 = (rng.uniform(0.5, 1.5, size=E) * 0.03).astype(np.float32)
    ws2 = (rng.uniform(0.5, 1.5, size=E) * 0.03).astype(np.float32)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int64)
    w = rng.random((T, k)).astype(np.float32)
    x_t = cuda(rng.standard_normal((T, hidden)).astype(np.float32), torch.float16)
    sentinel = torch.zeros(E, 1, 1, dtype=torch.int16, device="cuda")
    bl = lambda n: torch.tensor(O.block_decompose(n))
    y = ops.fused_moe_trellis_3inst(x_t, cuda(ids), cuda(w), cuda(w13), sentinel, cuda(su13), cuda(sv13), cuda(ws13),
                                    cuda(ws13), cuda(w2), sentinel, cuda(su2), cuda(sv2), cuda(ws2), cuda(ws2),
                                    hidden, inter, inter, hidden, inter, inter, hidden,
                                    bl(hidden), bl(inter), None, None, bl(inter), bl(hidden), None, None, act)
    f16 = lambda a: a.astype(np.float16).astype(np.float32)
    W13 = [CO.trellis_decode(w13[e], inter, hidden, 4).astype(np.float32) for e in range(E)]
    W2 = [CO.trellis_decode(w2[e], hidden, inter, 4).astype(np.float32) for e in range(E)]
    f13 = lambda e, xb: f16(O.linear_forward(xb, W13[e], su13[e], sv13, float(ws13[e])))
    f2 = lambda e, hb: f16(O.linear_forward(f16(hb), W2[e], su2[e], sv2, float(ws2[e])))
    ref = O.moe_forward(x_t.float().cpu().numpy(), ids, w, f13, f2, inter, O.ACT_CODES[act])
    assert relerr(y.float().cpu().numpy(), ref) <= MOE_TOL
    ops.clear_caches()


# ---------------------------------------------------------------------------------------------------------
# E8-shell experts: fused_moe_grouped_gemm / fused_moe_block_diag
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("stages", [1, 2, 3])
@pytest.mark.parametrize("T,act", [(1, 0), (9, 1), (200, 1), (33, 4)])
def test_e8_moe_vs_oracle(ops, packed_table, cb16, stages, T, act):
    E, hidden, inter, k = 8, 256, 128, 2
    gated = act < 3
    w13_out = 2 * inter if gated else inter
    rng = np.random.default_rng(5000 + stages * 100 + T + act)
    q13 = [idx(rng, E, w13_out, hidden // 8) for _ in range(stages)]
    q2 = [idx(rng, E, hidden, inter // 8) for _ in range(stages)]
    inv13 = [(rng.uniform(0.05, 0.3, size=E)).astype(np.float32) for _ in range(stages - 1)]
    inv2 = [(rng.uniform(0.05, 0.3, size=E)).astype(np.float32) for _ in range(stages - 1)]
    su13, sv13, su2, sv2 = signs(rng, E, w13_out), signs(rng, hidden), signs(rng, E, hidden), signs(rng, inter)
    ws13 = (rng.uniform(0.5, 1.5, size=E) * 0.03).astype(np.float32)
    ws2 = (rng.uniform(0.5, 1.5, size=E) * 0.03).astype(np.float32)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int64)
    if T > 3:
        ids[2, 1] = -1                                   # a routing that belongs to another rank
    w = rng.random((T, k)).astype(np.float32)
    x_t = cuda(rng.standard_normal((T, hidden)).astype(np.float32), torch.float16)
    placeholder = torch.zeros(E, 1, 1, dtype=torch.int16, device="cuda")
    zeros_e = torch.zeros(E, dtype=torch.float32, device="cuda")
    bl = lambda n: torch.tensor(O.block_decompose(n))
    st = lambda lst, s, alt: cuda(lst[s]) if s < len(lst) else alt
    args = (x_t, cuda(ids), cuda(w),
            cuda(q13[0]), cuda(su13), cuda(sv13), cuda(ws13), st(q13, 1, placeholder), st(inv13, 0, zeros_e),
            cuda(q2[0]), cuda(su2), cuda(sv2), cuda(ws2), st(q2, 1, placeholder), st(inv2, 0, zeros_e),
            cb16, cb16, hidden, inter, w13_out, hidden, w13_out, inter, hidden,
            bl(hidden), bl(w13_out), None, None, bl(inter), bl(hidden), None, None, act,
            st(q13, 2, placeholder), st(inv13, 1, zeros_e), st(q2, 2, placeholder), st(inv2, 1, zeros_e), cb16)
    y = ops.fused_moe_grouped_gemm(*args)
    assert torch.equal(y, ops.fused_moe_block_diag(*args))           # same op behind both names, deterministic
    f16 = lambda a: a.astype(np.float16).astype(np.float32)

    def dec(qs, invs, e, m, n):
        return CO.e8_decode([q[e] for q in qs], [packed_table] * stages, [float(v[e]) for v in invs], m, n)
    W13 = [dec(q13, inv13, e, w13_out, hidden) for e in range(E)]
    W2 = [dec(q2, inv2, e, hidden, inter) for e in range(E)]
    f13 = lambda e, xb: f16(O.linear_forward(xb, W13[e], su13[e], sv13, float(ws13[e])))
    f2 = lambda e, hb: f16(O.linear_forward(f16(hb), W2[e], su2[e], sv2, float(ws2[e])))
    keep = ids >= 0
    ref = O.moe_forward(x_t.float().cpu().numpy(), np.where(keep, ids, 0), np.where(keep, w, 0.0).astype(np.float32),
                        f13, f2, inter, O.ACT_CODES[act])
    assert relerr(y.float().cpu().numpy(), ref) <= MOE_TOL
    ops.clear_caches()


# ---------------------------------------------------------------------------------------------------------
# smaller gaps
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("stages", [1, 2])
@pytest.mark.parametrize("T", [1, 100, 300])
def test_e8_index_rows_that_are_not_16_byte_aligned(ops, packed_table, cb16, stages, T):
    """n = 200: 25 indices (50 bytes) per row, so rows start on 2-byte boundaries only; every vector-load path
    (streaming, fused GEMM producers, tile decode) has to take its scalar branch."""
    m, n = 320, 200
    rng = np.random.default_rng(200 + stages + T)
    qs, inv, W, su, sv, ws = _e8_layer(rng, m, n, stages, packed_table)
    x_t = cuda(rng.standard_normal((T, n)).astype(np.float32), torch.float16)
    y = _run_e8(ops, x_t, qs, inv, su, sv, ws, m, n, cb16)
    ref = O.linear_forward(x_t.float().cpu().numpy(), W, su, sv, ws)
    assert relerr(y.cpu().numpy(), ref) <= TOL
    ops.clear_caches()


def test_trellis_yrht_rvq2_two_shards(ops):
    """Two-stage shards stopped before the output transform, then one transform over both (the offsets in
    column 0 of the meta are honoured: the shards are deposited in swapped order)."""
    rng = np.random.default_rng(81)
    n, ms, B = 256, [64, 96], 3
    x = cuda(rng.standard_normal((B, n)).astype(np.float32))
    y_rht = torch.zeros(B, sum(ms), dtype=torch.float32, device="cuda")
    cols = [96, 0]                                       # shard 0 lives at columns 96.., shard 1 at 0..
    su_all = np.zeros(sum(ms), dtype=np.float16)
    meta, refs = [], []
    for m, col in zip(ms, cols):
        p1, p2 = idx(rng, (m // 16) * (n // 16), 64), idx(rng, (m // 16) * (n // 16), 32)
        su, sv, ws, inv = signs(rng, m), signs(rng, n), 0.03, 0.21
        W = CO.trellis_decode_f32(p1, 4, p2, 2, inv, m, n)
        ops.fused_linear_trellis_3inst_yrht_rvq2(x, cuda(sv), cuda(p1), cuda(p2), torch.tensor(O.block_decompose(n)),
                                                 None, ws, inv, n, n, m, y_rht, col)
        off = col
        for bs in O.block_decompose(m):
            meta.append([off, bs, int(np.log2(bs)), 0])
            off += bs
        su_all[col:col + m] = su
        refs.append((col, m, O.linear_forward(x.cpu().numpy(), W, su, sv, ws)))
    y = torch.empty(B, sum(ms), dtype=torch.float32, device="cuda")
    ops.output_rht_shards(y_rht, cuda(su_all), y, sum(ms), torch.tensor(meta, dtype=torch.int32, device="cuda"), 64)
    for col, m, ref in refs:
        assert relerr(y[:, col:col + m].cpu().numpy(), ref) <= TOL


def test_stateless_c_entry_point(packed_table):
    """glqb_fused_linear with a workspace of glqb_linear_workspace_bytes, trellis and E8 (3 tokens: the E8
    activations are padded to 8 tokens inside), straight through the C ABI."""
    from glq_b200 import _lib
    from glq_b200.plan import LinearSpec
    lib = _lib.load()
    rng = np.random.default_rng(31)
    m, n, B = 352, 576, 3
    x = cuda(rng.standard_normal((B, n)).astype(np.float32))
    su, sv = signs(rng, m), signs(rng, n)
    su_t, sv_t = cuda(su), cuda(sv)
    packed = idx(rng, (m // 16) * (n // 16), 64)
    qs = [idx(rng, m, n // 8) for _ in range(2)]
    tab = cuda(packed_table.view(np.int32))
    cases = [
        (LinearSpec(format=_lib.FMT_TRELLIS_3INST, m_pad=m, n_pad=n, in_features=n, out_features=m, codes=[cuda(packed)],
                    bits=[4], su=su_t, sv=sv_t, wscale=0.02, batch=B, x_dtype=torch.float32, y_dtype=torch.float32),
         CO.trellis_decode(packed, m, n, 4).astype(np.float32)),
        (LinearSpec(format=_lib.FMT_E8_SHELL, m_pad=m, n_pad=n, in_features=n, out_features=m, codes=[cuda(q) for q in qs],
                    tables=[tab, tab], stage_scale=[0.1], su=su_t, sv=sv_t, wscale=0.02, batch=B,
                    x_dtype=torch.float32, y_dtype=torch.float32),
         CO.e8_decode(qs, [packed_table] * 2, [0.1], m, n)),
    ]
    for spec, W in cases:
        d = spec.to_desc()
        nbytes = lib.glqb_linear_workspace_bytes(C.byref(d))
        ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        y = torch.empty(B, m, dtype=torch.float32, device="cuda")
        rc = lib.glqb_fused_linear(C.byref(d), x.data_ptr(), y.data_ptr(), ws.data_ptr(), nbytes,
                                   torch.cuda.current_stream().cuda_stream)
        assert rc == 0, lib.glqb_last_error()
        assert relerr(y.cpu().numpy(), O.linear_forward(x.cpu().numpy(), W, su, sv, 0.02)) <= TOL


def test_varying_token_counts_build_a_bounded_number_of_plans(ops):
    rng = np.random.default_rng(41)
    m, n = 128, 256
    packed = idx(rng, (m // 16) * (n // 16), 64)
    W = CO.trellis_decode(packed, m, n, 4).astype(np.float32)
    su, sv = signs(rng, m), signs(rng, n)
    t = dict(p=cuda(packed), su=cuda(su), sv=cuda(sv))
    ops.clear_caches()
    x = cuda(rng.standard_normal((700, n)).astype(np.float32))
    ref = O.linear_forward(x.cpu().numpy(), W, su, sv, 0.02)
    counts = [1, 3, 9, 10, 11, 17, 40, 63, 65, 70, 99, 130, 131, 200, 257, 300, 333, 511, 513, 700]
    for B in counts:
        y = ops.fused_linear_trellis_3inst(x[:B], t["sv"], t["su"], t["p"], None, None, None, None, 0.02, n, m, n, m)
        assert y.shape == (B, m)
        assert relerr(y.cpu().numpy(), ref[:B]) <= TOL, B
    assert len(ops._PLAN_CACHE) <= 11, len(ops._PLAN_CACHE)      # 1, 3, 16, 24, 40, 64, 128, 256, 512, 768
    assert len(ops._WORKSPACES) == 1                             # one shared workspace on this stream
    ops.check_device_status()
    ops.clear_caches()


def test_dequantize_matches_forward(ops, packed_table, cb16):
    from glq_b200.linear import GLQLinear
    rng = np.random.default_rng(51)
    lt = GLQLinear(576, 352, codebook_type="trellis").cuda()
    lt.trellis_packed = cuda(idx(rng, (352 // 16) * (576 // 16), 64))
    lt.SU, lt.SV = cuda(signs(rng, 352)), cuda(signs(rng, 576))
    lt.Wscale = torch.tensor(0.03, device="cuda")
    le = GLQLinear(200, 96, block_diagonal=True).cuda()
    le.Qidxs, le.Qidxs2 = cuda(idx(rng, 96, 25)), cuda(idx(rng, 96, 25))
    le.SU, le.SV = cuda(signs(rng, 96)), cuda(signs(rng, 200))
    le.Wscale = torch.tensor(0.02, device="cuda")
    le.inv_resid_scale = torch.tensor(0.1, device="cuda")
    le.set_codebook(cb16, cb16)
    for layer in (lt, le):
        W = layer.dequantize()
        assert W.shape == (layer.out_features, layer.in_features) and W.dtype == torch.float32
        x = torch.randn(4, layer.in_features, device="cuda")
        y = layer(x)
        ref = x @ W.t()
        assert ((y - ref).abs().max() / ref.abs().max()).item() <= TOL
    # against the oracle's definition as well (trellis layer)
    Wrot = CO.trellis_decode(lt.trellis_packed.cpu().numpy(), 352, 576, 4).astype(np.float32)
    eye = np.eye(576, dtype=np.float32)
    Wd = O.linear_forward(eye, Wrot, lt.SU.cpu().numpy(), lt.SV.cpu().numpy(), 0.03).T
    assert relerr(lt.dequantize().cpu().numpy(), Wd) <= 1e-5
    ops.clear_caches()


def test_unfused_transforms_are_capturable_and_exact(ops):
    """input_rht / output_rht allocate nothing and copy nothing from the host: they can be captured into a CUDA
    graph, and the replayed graph gives the oracle's transform."""
    rng = np.random.default_rng(61)
    B, n, n_pad = 6, 1000, 1024
    x = cuda(rng.standard_normal((B, n)).astype(np.float32), torch.float16)
    sv, su = signs(rng, n_pad), signs(rng, n_pad)
    sv_t, su_t = cuda(sv), cuda(su)
    mid = torch.zeros(B, n_pad, dtype=torch.float32, device="cuda")
    out = torch.zeros(B, n, dtype=torch.float32, device="cuda")
    ops.input_rht(x, sv_t, mid, n, n, 1 / 32.0, n_pad, 10)         # first call outside capture (sets kernel limits)
    ops.output_rht(mid, su_t, out, n, n_pad, 10, 1 / 32.0)
    torch.cuda.synchronize()
    mid.zero_(); out.zero_()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        ops.input_rht(x, sv_t, mid, n, n, 1 / 32.0, n_pad, 10)
        ops.output_rht(mid, su_t, out, n, n_pad, 10, 1 / 32.0)
    g.replay()
    torch.cuda.synchronize()
    xp = np.zeros((B, n_pad), dtype=np.float32)
    xp[:, :n] = x.float().cpu().numpy()
    ref_mid = O.fht(xp * sv.astype(np.float32))
    assert relerr(mid.cpu().numpy(), ref_mid) <= 1e-5
    ref_out = (O.fht(ref_mid) * su.astype(np.float32))[:, :n]
    assert relerr(out.cpu().numpy(), ref_out) <= 1e-5


def test_large_block_plan_survives_a_later_smaller_plan(ops):
    """The shared-memory limit of the transform kernels belongs to the kernel, not to a plan: a plan with a
    32768-value Hadamard block must still launch after a plan with a 16384 block was built."""
    rng = np.random.default_rng(71)
    results = {}
    layers = {}
    for n in (32768, 16384):
        m = 64
        packed = idx(rng, (m // 16) * (n // 16), 32)
        su, sv = signs(rng, m), signs(rng, n)
        layers[n] = (packed, su, sv, cuda(rng.standard_normal((1, n)).astype(np.float32)),
                     cuda(packed), cuda(su), cuda(sv))          # fixed device tensors: the plan is built once

    def run(n):
        _, _, _, x, p_t, su_t, sv_t = layers[n]
        return ops.fused_linear_trellis_3inst(x, sv_t, su_t, p_t, None, None, None, None, 0.02, n, 64, n, 64)
    results[32768] = run(32768)
    run(16384)
    again = run(32768)
    torch.cuda.synchronize()
    assert torch.equal(again, results[32768])
    packed, su, sv, x = layers[32768][:4]
    W = CO.trellis_decode(packed, 64, 32768, 2).astype(np.float32)
    assert relerr(again.cpu().numpy(), O.linear_forward(x.cpu().numpy(), W, su, sv, 0.02)) <= TOL
    ops.clear_caches()


# ---------------------------------------------------------------------------------------------------------
# decoder-layer steps fused into the single-launch decode kernel: RMSNorm, act(gate) * up, residual add
# ---------------------------------------------------------------------------------------------------------
def _bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


@pytest.mark.parametrize("B", [1, 5, 20])
def test_fused_norm_activation_residual(ops, B):
    """Up to 8 tokens the three steps run inside the decode kernel, above that as torch kernels around it; both
    must equal the same steps done on the host (intermediate values rounded to bf16 as separate kernels would
    store them) followed by the oracle's linear."""
    rng = np.random.default_rng(7000 + B)
    m, n = 352, 576
    packed = idx(rng, (m // 16) * (n // 16), 64)
    W = CO.trellis_decode(packed, m, n, 4).astype(np.float32)
    su, sv, ws = signs(rng, m), signs(rng, n), 0.02
    t = dict(p=cuda(packed), su=cuda(su), sv=cuda(sv))
    call = lambda x, **kw: ops.fused_linear_trellis_3inst(x, t["sv"], t["su"], t["p"], None, None, None, None, ws,
                                                          n, m, n, m, **kw)
    x = cuda(rng.standard_normal((B, n)).astype(np.float32) * 3.0, torch.bfloat16)
    xf = x.float().cpu().numpy()
    # RMSNorm in front of the linear
    w = cuda(1.0 + 0.2 * rng.standard_normal(n).astype(np.float32), torch.bfloat16)
    eps = 1e-5
    y = call(x, in_norm_weight=w, in_norm_eps=eps, out_dtype=torch.float32)
    xn = _bf16(xf / np.sqrt((xf.astype(np.float64) ** 2).mean(-1, keepdims=True) + eps))
    xin = _bf16(w.float().cpu().numpy() * xn)
    assert relerr(y.cpu().numpy(), O.linear_forward(xin, W, su, sv, ws)) <= TOL + 2.0 ** -8
    # act(gate) * up in front of the linear, every gated activation
    xg = cuda(rng.standard_normal((B, 2 * n)).astype(np.float32), torch.bfloat16)
    g, u = xg.float().cpu().numpy()[:, :n], xg.float().cpu().numpy()[:, n:]
    for code in (0, 1, 2):
        y = call(xg, gated_act=code, out_dtype=torch.float32)
        xin = _bf16(_bf16(O._act(O.ACT_CODES[code])(g)) * u)
        assert relerr(y.cpu().numpy(), O.linear_forward(xin, W, su, sv, ws)) <= TOL + 2.0 ** -8, code
    # residual add behind the linear, in place
    res = cuda(rng.standard_normal((B, m)).astype(np.float32), torch.bfloat16)
    h = res.clone()
    out = call(x, accumulate_into=h)
    assert out.data_ptr() == h.data_ptr()
    ref = res.float().cpu().numpy() + O.linear_forward(xf, W, su, sv, ws)
    assert relerr(h.float().cpu().numpy(), ref) <= TOL + 2.0 ** -7
    # all three at once equal the same composition
    h2 = res.clone()
    call(xg, gated_act=0, accumulate_into=h2)
    xin = _bf16(_bf16(O._act("silu")(g)) * u)
    ref = res.float().cpu().numpy() + O.linear_forward(xin, W, su, sv, ws)
    assert relerr(h2.float().cpu().numpy(), ref) <= TOL + 2.0 ** -7
    ops.clear_caches()


@pytest.mark.parametrize("B,n", [(1, 576), (5, 576), (2, 4672)])
def test_fused_steps_in_the_three_launch_form(ops, monkeypatch, B, n):
    """With the single-launch form switched off the same steps are applied by the transform kernels (norm and
    activation by the input transform, the residual by the output transform); n = 4672 has a 4096-value Hadamard block,
    which several CTAs share."""
    monkeypatch.setenv("GLQB_FUSED_DECODE", "0")
    ops.clear_caches()
    rng = np.random.default_rng(7400 + B + n)
    m = 4128                                                   # 4096 + 32: a long output block as well
    packed = idx(rng, (m // 16) * (n // 16), 64)
    W = CO.trellis_decode(packed, m, n, 4).astype(np.float32)
    su, sv, ws = signs(rng, m), signs(rng, n), 0.02
    t = dict(p=cuda(packed), su=cuda(su), sv=cuda(sv))
    call = lambda x, **kw: ops.fused_linear_trellis_3inst(x, t["sv"], t["su"], t["p"], None, None, None, None, ws,
                                                          n, m, n, m, **kw)
    x = cuda(rng.standard_normal((B, n)).astype(np.float32) * 3.0, torch.bfloat16)
    xf = x.float().cpu().numpy()
    w = cuda(1.0 + 0.2 * rng.standard_normal(n).astype(np.float32), torch.bfloat16)
    eps = 1e-5
    res = cuda(rng.standard_normal((B, m)).astype(np.float32), torch.bfloat16)
    h = res.clone()
    call(x, in_norm_weight=w, in_norm_eps=eps, accumulate_into=h)
    plans = [p for p in ops._PLAN_CACHE.values() if hasattr(p, "launches")]
    assert plans and all(p.launches == 3 for p in plans)
    xn = _bf16(xf / np.sqrt((xf.astype(np.float64) ** 2).mean(-1, keepdims=True) + eps))
    xin = _bf16(w.float().cpu().numpy() * xn)
    ref = res.float().cpu().numpy() + O.linear_forward(xin, W, su, sv, ws)
    assert relerr(h.float().cpu().numpy(), ref) <= TOL + 2.0 ** -7
    xg = cuda(rng.standard_normal((B, 2 * n)).astype(np.float32), torch.bfloat16)
    g, u = xg.float().cpu().numpy()[:, :n], xg.float().cpu().numpy()[:, n:]
    y = call(xg, gated_act=1, out_dtype=torch.float32)
    xin = _bf16(_bf16(O._act(O.ACT_CODES[1])(g)) * u)
    assert relerr(y.cpu().numpy(), O.linear_forward(xin, W, su, sv, ws)) <= TOL + 2.0 ** -8
    ops.clear_caches()


@pytest.mark.parametrize("B", [1, 5, 20])
def test_fused_norm_activation_residual_e8(ops, packed_table, cb16, B):
    """The same three steps around an E8-shell layer (two stages, block-diagonal 320 x 576): inside the single-launch
    E8 kernel up to 8 tokens, as torch kernels around the linear above that."""
    rng = np.random.default_rng(7300 + B)
    m, n = 320, 576
    qs, inv, W, su, sv, ws = _e8_layer(rng, m, n, 2, packed_table)
    t = dict(q=[cuda(q) for q in qs], su=cuda(su), sv=cuda(sv))
    ei = torch.empty(0, dtype=torch.int16, device="cuda")
    eh = torch.empty(0, dtype=torch.float16, device="cuda")
    bn, bm = torch.tensor(O.block_decompose(n)), torch.tensor(O.block_decompose(m))
    call = lambda x, **kw: ops.fused_linear_block_diag(x, t["sv"], t["su"], t["q"][0], cb16, ws, n, m, n, m, bn, bm, None, None,
                                                       t["q"][1], cb16, inv[0], ei, eh, 0.0, ei, eh, 0.0, **kw)
    x = cuda(rng.standard_normal((B, n)).astype(np.float32) * 3.0, torch.bfloat16)
    xf = x.float().cpu().numpy()
    w = cuda(1.0 + 0.2 * rng.standard_normal(n).astype(np.float32), torch.bfloat16)
    eps = 1e-5
    y = call(x, in_norm_weight=w, in_norm_eps=eps, out_dtype=torch.float32)
    xn = _bf16(xf / np.sqrt((xf.astype(np.float64) ** 2).mean(-1, keepdims=True) + eps))
    xin = _bf16(w.float().cpu().numpy() * xn)
    assert relerr(y.cpu().numpy(), O.linear_forward(xin, W, su, sv, ws)) <= TOL + 2.0 ** -8
    xg = cuda(rng.standard_normal((B, 2 * n)).astype(np.float32), torch.bfloat16)
    g, u = xg.float().cpu().numpy()[:, :n], xg.float().cpu().numpy()[:, n:]
    res = cuda(rng.standard_normal((B, m)).astype(np.float32), torch.bfloat16)
    h = res.clone()
    out = call(xg, gated_act=0, accumulate_into=h)
    assert out.data_ptr() == h.data_ptr()
    xin = _bf16(_bf16(O._act("silu")(g)) * u)
    ref = res.float().cpu().numpy() + O.linear_forward(xin, W, su, sv, ws)
    assert relerr(h.float().cpu().numpy(), ref) <= TOL + 2.0 ** -7
    if B <= 8:
        plans = [p for p in ops._PLAN_CACHE.values() if hasattr(p, "launches")]
        assert plans and all(p.launches == 1 for p in plans)
    ops.clear_caches()


def test_fused_norm_on_shards_in_one_launch(ops):
    rng = np.random.default_rng(7100)
    n, ms = 2048, [2048, 512, 512]
    sv = signs(rng, n)
    shards, refs = [], []
    x = cuda(rng.standard_normal((1, n)).astype(np.float32) * 2.0, torch.bfloat16)
    w = cuda(1.0 + 0.1 * rng.standard_normal(n).astype(np.float32), torch.float32)
    xf = x.float().cpu().numpy()
    xn = _bf16(xf / np.sqrt((xf.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6))
    xin = _bf16(w.cpu().numpy() * xn)
    for m in ms:
        packed = idx(rng, (m // 16) * (n // 16), 64)
        su = signs(rng, m)
        shards.append((cuda(su), cuda(packed), None, 0.02, 0.0, m))
        refs.append(O.linear_forward(xin, CO.trellis_decode(packed, m, n, 4).astype(np.float32), su, sv, 0.02))
    y = ops.fused_linear_trellis_3inst_shards(x, cuda(sv), shards, out_dtype=torch.float32, in_norm_weight=w, in_norm_eps=1e-6)
    plan = [p for k, p in ops._PLAN_CACHE.items() if k[0] == "trellis_shards"][0]
    assert plan.launches == 1
    assert relerr(y.cpu().numpy(), np.concatenate(refs, axis=1)) <= TOL + 2.0 ** -8
    ops.clear_caches()
