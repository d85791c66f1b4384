"""MoE grouped expert matmul on the GPU against the CPU oracle (per-expert decode + dense loop)."""
import numpy as np
import pytest
import torch

from oracle import glq_oracle as O

pytestmark = pytest.mark.gpu


def cuda(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def _make(rng, E, hidden, inter, K, K2=0):
    w13_out = 2 * inter
    def packed(m, n, k):
        return rng.integers(0, 65536, size=(E, (m // 16) * (n // 16), 16 * k), dtype=np.uint16).view(np.int16)
    sg = lambda *s: (rng.integers(0, 2, size=s) * 2 - 1).astype(np.float16)
    d = dict(w13=packed(w13_out, hidden, K), w2=packed(hidden, inter, K),
             w13_2=packed(w13_out, hidden, K2) if K2 else None, w2_2=packed(hidden, inter, K2) if K2 else None,
             su13=sg(E, w13_out), sv13=sg(hidden), su2=sg(E, hidden), sv2=sg(inter),
             ws13=(rng.uniform(0.5, 1.5, size=E) * 0.03).astype(np.float32),
             ws2=(rng.uniform(0.5, 1.5, size=E) * 0.03).astype(np.float32),
             inv13=np.full(E, 0.2, np.float32), inv2=np.full(E, 0.15, np.float32))
    return d, w13_out


def _oracle(d, x, ids, w, E, hidden, inter, w13_out, K, K2, act):
    W13, W2 = {}, {}
    def dec(p, p2, inv, e, m, n):
        if K2:
            return O.trellis_decode_layer_nstage([p[e], p2[e]], [K, K2], [1.0, float(inv[e])], m, n)
        return O.trellis_decode_layer(p[e], m, n, K).astype(np.float32)
    def f13(e, xb):
        if e not in W13:
            W13[e] = dec(d["w13"], d["w13_2"], d["inv13"], e, w13_out, hidden)
        y = O.linear_forward(xb, W13[e], d["su13"][e], d["sv13"], float(d["ws13"][e]))
        return y.astype(np.float16).astype(np.float32)
    def f2(e, hb):
        if e not in W2:
            W2[e] = dec(d["w2"], d["w2_2"], d["inv2"], e, hidden, inter)
        hb = hb.astype(np.float16).astype(np.float32)
        return O.linear_forward(hb, W2[e], d["su2"][e], d["sv2"], float(d["ws2"][e])).astype(np.float16).astype(np.float32)
    return O.moe_forward(x, ids, w, f13, f2, inter, act)


def _run(ops, d, x_t, ids_t, w_t, E, hidden, inter, w13_out, K2, act_code):
    sentinel = torch.zeros(E, 1, 1, dtype=torch.int16, device="cuda")
    bl = lambda n: torch.tensor(O.block_decompose(n))
    return ops.fused_moe_trellis_3inst(
        x_t, ids_t, w_t,
        cuda(d["w13"]), cuda(d["w13_2"]) if K2 else sentinel, cuda(d["su13"]), cuda(d["sv13"]), cuda(d["ws13"]), cuda(d["inv13"]),
        cuda(d["w2"]), cuda(d["w2_2"]) if K2 else sentinel, cuda(d["su2"]), cuda(d["sv2"]), cuda(d["ws2"]), cuda(d["inv2"]),
        hidden, inter, w13_out, hidden, w13_out, inter, hidden,
        bl(hidden), bl(w13_out), None, None, bl(inter), bl(hidden), None, None, act_code)


@pytest.mark.parametrize("K,K2", [(4, 0), (2, 0), (4, 2)])
@pytest.mark.parametrize("T,act", [(1, 1), (7, 0), (40, 1), (40, 2)])
def test_moe_vs_oracle(K, K2, T, act):
    from glq_b200 import ops
    E, hidden, inter, k = 8, 256, 96, 2
    rng = np.random.default_rng(K * 100 + K2 * 10 + T + act)
    d, w13_out = _make(rng, E, hidden, inter, K, K2)
    x = rng.standard_normal((T, hidden)).astype(np.float32)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int64)
    w = rng.random((T, k)).astype(np.float32)
    w /= w.sum(1, keepdims=True)
    x_t = cuda(x, torch.float16)
    y = _run(ops, d, x_t, cuda(ids), cuda(w), E, hidden, inter, w13_out, K2, act)
    ref = _oracle(d, x_t.float().cpu().numpy(), ids, w, E, hidden, inter, w13_out, K, K2, O.ACT_CODES[act])
    err = np.abs(y.float().cpu().numpy() - ref).max() / np.abs(ref).max()
    assert err <= 5e-3, err      # two chained layers with fp16 hand-offs (the reference's own gate is rtol=atol=2e-2)
    y2 = _run(ops, d, x_t, cuda(ids), cuda(w), E, hidden, inter, w13_out, K2, act)
    assert torch.equal(y, y2)


def test_moe_skewed_routing_and_int32_ids():
    """Everything routed to two experts (many decode passes for one expert, empty experts elsewhere)."""
    from glq_b200 import ops
    E, hidden, inter, k, T = 16, 128, 64, 2, 70
    rng = np.random.default_rng(3)
    d, w13_out = _make(rng, E, hidden, inter, 4)
    x = rng.standard_normal((T, hidden)).astype(np.float32)
    ids = np.tile(np.array([[3, 11]], dtype=np.int64), (T, 1))
    w = rng.random((T, k)).astype(np.float32)
    x_t = cuda(x, torch.bfloat16)
    y = _run(ops, d, x_t, cuda(ids.astype(np.int32)), cuda(w), E, hidden, inter, w13_out, 0, 1)
    ref = _oracle(d, x_t.float().cpu().numpy(), ids, w, E, hidden, inter, w13_out, 4, 0, "gelu_tanh")
    err = np.abs(y.float().cpu().numpy() - ref).max() / np.abs(ref).max()
    assert err <= 5e-3 + 2.0 ** -8, err


def test_moe_expert_roll_invariance():
    """Renaming the experts (rolling the stacked weights and the ids together) changes nothing."""
    from glq_b200 import ops
    E, hidden, inter, k, T = 8, 128, 64, 2, 9
    rng = np.random.default_rng(5)
    d, w13_out = _make(rng, E, hidden, inter, 4)
    x_t = cuda(rng.standard_normal((T, hidden)).astype(np.float32), torch.float16)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int64)
    w = cuda(rng.random((T, k)).astype(np.float32))
    y = _run(ops, d, x_t, cuda(ids), w, E, hidden, inter, w13_out, 0, 0)
    d2 = {kk: (np.roll(v, 3, axis=0) if isinstance(v, np.ndarray) and v.shape[:1] == (E,) else v) for kk, v in d.items()}
    y2 = _run(ops, d2, x_t, cuda((ids + 3) % E), w, E, hidden, inter, w13_out, 0, 0)
    assert torch.equal(y, y2)


@pytest.mark.parametrize("K,K2", [(4, 0), (3, 0), (4, 2)])
@pytest.mark.parametrize("T,skew", [(200, False), (333, True)])
def test_moe_tensor_core_form(K, K2, T, skew, monkeypatch):
    """Many routed tokens per expert: both matmuls run on the tcgen05 GEMM kernel over a device-built work
    list.  Checked against the oracle, for determinism, and against the streaming form of the same step."""
    from glq_b200 import ops
    E, hidden, inter, k = 8, 256, 128, 2
    rng = np.random.default_rng(7000 + K * 100 + K2 * 10 + T)
    d, w13_out = _make(rng, E, hidden, inter, K, K2)
    x = rng.standard_normal((T, hidden)).astype(np.float32)
    if skew:      # two hot experts take most routings, one expert gets none
        p = np.array([0.45, 0.35, 0.05, 0.05, 0.04, 0.03, 0.03, 0.0])
        ids = np.stack([rng.choice(E, size=k, replace=False, p=p) for _ in range(T)]).astype(np.int64)
    else:
        ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int64)
    w = rng.random((T, k)).astype(np.float32)
    w /= w.sum(1, keepdims=True)
    x_t = cuda(x, torch.float16)
    ref = _oracle(d, x_t.float().cpu().numpy(), ids, w, E, hidden, inter, w13_out, K, K2, O.ACT_CODES[1])
    outs = {}
    for form, min_avg in (("gemm", "1"), ("stream", "1000000")):
        monkeypatch.setenv("GLQB_MOE_GEMM_MIN_AVG", min_avg)
        ops.clear_caches()
        y = _run(ops, d, x_t, cuda(ids), cuda(w), E, hidden, inter, w13_out, K2, 1)
        y2 = _run(ops, d, x_t, cuda(ids), cuda(w), E, hidden, inter, w13_out, K2, 1)
        assert torch.equal(y, y2), form
        err = np.abs(y.float().cpu().numpy() - ref).max() / np.abs(ref).max()
        assert err <= 5e-3, (form, err)
        outs[form] = y.float()
    ops.clear_caches()
    # same math, different summation order (and one fp16 rounding of the folded second stage)
    rel = (outs["gemm"] - outs["stream"]).abs().max() / outs["stream"].abs().max()
    assert rel <= 4e-3, rel


def test_moe_zero_tokens_and_unrouted_tokens():
    """No tokens: empty result.  Routings with id -1 (what expert parallelism leaves for other ranks' experts)
    are skipped; a token whose routings are all skipped gets zeros."""
    from glq_b200 import ops
    E, hidden, inter, k = 8, 256, 96, 2
    rng = np.random.default_rng(4242)
    d, w13_out = _make(rng, E, hidden, inter, 4, 0)
    x0 = torch.zeros(0, hidden, dtype=torch.float16, device="cuda")
    y0 = _run(ops, d, x0, torch.zeros(0, k, dtype=torch.int64, device="cuda"),
              torch.zeros(0, k, dtype=torch.float32, device="cuda"), E, hidden, inter, w13_out, 0, 1)
    assert y0.shape == (0, hidden)
    T = 6
    x = rng.standard_normal((T, hidden)).astype(np.float32)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int64)
    w = rng.random((T, k)).astype(np.float32)
    x_t = cuda(x, torch.float16)
    full = _run(ops, d, x_t, cuda(ids), cuda(w), E, hidden, inter, w13_out, 0, 1).float()
    masked = ids.copy()
    masked[2, :] = -1                      # token 2: nothing routed here
    masked[4, 1] = -1                      # token 4: only its first routing
    y = _run(ops, d, x_t, cuda(masked), cuda(w), E, hidden, inter, w13_out, 0, 1).float()
    assert torch.count_nonzero(y[2]) == 0
    keep = [0, 1, 3, 5]
    assert torch.equal(y[keep], full[keep])
    only_first = ids.copy(); only_first[:, 1] = -1
    y_first = _run(ops, d, x_t, cuda(only_first), cuda(w), E, hidden, inter, w13_out, 0, 1).float()
    assert torch.equal(y[4], y_first[4])


def test_moe_large_step_uses_split_grouping():
    """More than 8192 routings: counting and placement run as many-CTA kernels around the table-building CTA."""
    from glq_b200 import ops
    E, hidden, inter, k, T = 8, 256, 128, 2, 4200
    rng = np.random.default_rng(9001)
    d, w13_out = _make(rng, E, hidden, inter, 4, 0)
    x = rng.standard_normal((T, hidden)).astype(np.float32)
    p = np.array([0.3, 0.25, 0.15, 0.1, 0.08, 0.07, 0.05, 0.0])
    ids = np.stack([rng.choice(E, size=k, replace=False, p=p) for _ in range(T)]).astype(np.int64)
    ids[17, 0] = -1                                   # a skipped routing in the middle
    w = rng.random((T, k)).astype(np.float32)
    w /= w.sum(1, keepdims=True)
    x_t = cuda(x, torch.float16)
    ops.clear_caches()
    y = _run(ops, d, x_t, cuda(ids), cuda(w), E, hidden, inter, w13_out, 0, 1)
    y2 = _run(ops, d, x_t, cuda(ids), cuda(w), E, hidden, inter, w13_out, 0, 1)
    assert torch.equal(y, y2)
    keep = ids >= 0
    ref = _oracle(d, x_t.float().cpu().numpy(), np.where(keep, ids, 7), np.where(keep, w, 0.0).astype(np.float32),
                  E, hidden, inter, w13_out, 4, 0, O.ACT_CODES[1])
    err = np.abs(y.float().cpu().numpy() - ref).max() / np.abs(ref).max()
    assert err <= 5e-3, err
    ops.clear_caches()
