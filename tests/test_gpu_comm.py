"""The in-kernel sum over tensor-parallel ranks (glqb_comm_*, glqb_plan_set_comm) on ONE GPU.

Two ranks of one communicator live in this process, both on cuda:0.  Kernels that wait for one another must never
share a GPU, so the ranks run one after the other: the rank that goes first stores its pieces and raises its flags,
then finds nothing from its peer and gives up after a few milliseconds (status 6, checked here: that is the
bounded-wait test); the rank that goes second finds the first one's flags already raised, never waits, and must
produce the exact fixed-order sum.  The order of the ranks alternates between passes, which also exercises the
double-buffered receive areas.  The real multi-GPU run of the same kernels is `bench.py --gpus N`.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle import c_oracle as CO
from oracle import glq_oracle as O

pytestmark = pytest.mark.gpu
TOL = 2e-3


def cuda(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t.to(dtype) if dtype is not None else t


def relerr(y, ref):
    y, ref = np.asarray(y, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    return np.abs(y - ref).max() / max(np.abs(ref).max(), 1e-30)


@pytest.fixture()
def pair():
    from glq_b200.comm import Comm
    comms = Comm.local_group(2, max_floats=1 << 15)
    for c in comms:
        c.set_timeout_ms(20)
    yield comms
    torch.cuda.synchronize()
    for c in comms:
        c.close()


def test_all_reduce_fixed_order_and_bounded_wait(pair):
    rng = np.random.default_rng(1)
    for round_, count in enumerate([5000, 1 << 15, 37, 4096]):
        a = rng.standard_normal(count).astype(np.float32)
        b = rng.standard_normal(count).astype(np.float32)
        bufs = [cuda(a), cuda(b)]
        first = round_ & 1                         # the rank that runs first finds no peer and must give up
        second = 1 - first
        pair[first].all_reduce_(bufs[first])
        torch.cuda.synchronize()
        assert pair[first].status() == 6
        with pytest.raises(RuntimeError, match=r"code -4"):
            pair[first].check_status()
        assert pair[first].status(reset=True) == 6 and pair[first].status() == 0
        pair[second].all_reduce_(bufs[second])
        torch.cuda.synchronize()
        assert pair[second].status() == 0
        assert np.array_equal(bufs[second].cpu().numpy(), a + b)          # rank order 0, 1: a + b, bit for bit
        assert pair[0].epoch() == pair[1].epoch() == round_ + 1


def test_all_reduce_rejects_what_does_not_fit(pair):
    big = torch.zeros((1 << 15) + 4, device="cuda")
    with pytest.raises(RuntimeError, match="communicator holds"):
        pair[0].all_reduce_(big)
    with pytest.raises(RuntimeError):
        pair[0].all_reduce_(torch.zeros(8, device="cuda", dtype=torch.float16))


def _shard(rng, m, n):
    packed = rng.integers(0, 65536, size=((m // 16) * (n // 16), 64), dtype=np.uint16).view(np.int16)
    W = CO.trellis_decode(packed, m, n, 4).astype(np.float32)
    su = (rng.integers(0, 2, size=m) * 2 - 1).astype(np.float16)
    sv = (rng.integers(0, 2, size=n) * 2 - 1).astype(np.float16)
    return dict(p=cuda(packed), su=cuda(su), sv=cuda(sv), W=W, su_h=su, sv_h=sv, ws=float(0.01 + 0.02 * rng.random()))


@pytest.mark.parametrize("B,m,n", [(1, 2048, 1024), (3, 352, 576), (8, 2048 + 512, 2048)])
def test_row_parallel_linear_summed_inside_the_decode_kernel(pair, B, m, n):
    """Each rank holds its own column shard (own codes, signs and scale) of a row-parallel layer and its own slice
    of the input; with ``reduce_over`` the single-launch kernel leaves, on the rank that runs second, the sum of
    both ranks' outputs (plus the residual): compared with the oracle's two linears added on the host."""
    from glq_b200 import ops
    rng = np.random.default_rng(100 + B)
    sh = [_shard(rng, m, n), _shard(rng, m, n)]
    xs = [cuda(rng.standard_normal((B, n)).astype(np.float32), torch.bfloat16) for _ in range(2)]
    res = cuda(rng.standard_normal((B, m)).astype(np.float32), torch.bfloat16)
    refs = [O.linear_forward(xs[r].float().cpu().numpy(), sh[r]["W"], sh[r]["su_h"], sh[r]["sv_h"], sh[r]["ws"]) for r in range(2)]
    total = refs[0].astype(np.float64) + refs[1].astype(np.float64)

    def call(r, **kw):
        s = sh[r]
        return ops.fused_linear_trellis_3inst(xs[r], s["sv"], s["su"], s["p"], None, None, None, None, s["ws"],
                                              n, m, n, m, reduce_over=pair[r], **kw)

    launches0 = pair[0].epoch()
    # first pass: rank 1 first (gives up), rank 0 second (complete sum), fp32 output
    call(1, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert pair[1].status(reset=True) == 6
    y0 = call(0, out_dtype=torch.float32)
    torch.cuda.synchronize()
    assert pair[0].status() == 0
    assert relerr(y0.cpu().numpy(), total) <= TOL
    # the sum is taken in rank order over each rank's own fp32 result: equal to adding the two single-rank outputs
    y_single = [ops.fused_linear_trellis_3inst(xs[r], sh[r]["sv"], sh[r]["su"], sh[r]["p"], None, None, None, None,
                                               sh[r]["ws"], n, m, n, m, out_dtype=torch.float32) for r in range(2)]
    assert torch.equal(y0, y_single[0] + y_single[1])
    # second pass: rank 0 first, rank 1 second, with the residual add
    h = [res.clone(), res.clone()]
    call(0, accumulate_into=h[0])
    torch.cuda.synchronize()
    assert pair[0].status(reset=True) == 6
    out = call(1, accumulate_into=h[1])
    torch.cuda.synchronize()
    assert pair[1].status() == 0 and out.data_ptr() == h[1].data_ptr()
    assert relerr(h[1].float().cpu().numpy(), res.float().cpu().numpy() + total) <= TOL + 2.0 ** -7
    # one launch that used the communicator per call and rank (the kernel itself counts them)
    assert pair[0].epoch() == pair[1].epoch() == launches0 + 2
    ops.clear_caches()


def test_row_parallel_e8_linear_summed_inside_the_decode_kernel(pair):
    """The same sum inside the single-launch E8 kernel (two-stage shards of 320 x 576, 2 tokens)."""
    import os
    from glq_b200 import ops
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    table = np.load(os.path.join(root, "glq_b200", "data", "e8_shell_packed.npy"))
    cb = cuda(O.e8_unpack_table(table).astype(np.float16))
    rng = np.random.default_rng(77)
    B, m, n = 2, 320, 576
    ei = torch.empty(0, dtype=torch.int16, device="cuda")
    eh = torch.empty(0, dtype=torch.float16, device="cuda")
    bn, bm = torch.tensor(O.block_decompose(n)), torch.tensor(O.block_decompose(m))
    sh, refs, xs = [], [], []
    for r in range(2):
        qs = [rng.integers(0, 65536, size=(m, n // 8), dtype=np.uint16).view(np.int16) for _ in range(2)]
        su = (rng.integers(0, 2, size=m) * 2 - 1).astype(np.float16)
        sv = (rng.integers(0, 2, size=n) * 2 - 1).astype(np.float16)
        W = CO.e8_decode(qs, [table, table], [0.1], m, n)
        x = cuda(rng.standard_normal((B, n)).astype(np.float32), torch.bfloat16)
        sh.append(dict(q=[cuda(q) for q in qs], su=cuda(su), sv=cuda(sv)))
        xs.append(x)
        refs.append(O.linear_forward(x.float().cpu().numpy(), W, su, sv, 0.02))
    call = lambda r: ops.fused_linear_block_diag(xs[r], sh[r]["sv"], sh[r]["su"], sh[r]["q"][0], cb, 0.02, n, m, n, m, bn, bm,
                                                 None, None, sh[r]["q"][1], cb, 0.1, ei, eh, 0.0, ei, eh, 0.0,
                                                 out_dtype=torch.float32, reduce_over=pair[r])
    e0 = pair[0].epoch()
    call(1)
    torch.cuda.synchronize()
    assert pair[1].status(reset=True) == 6
    y = call(0)
    torch.cuda.synchronize()
    assert pair[0].status() == 0 and pair[0].epoch() == e0 + 1          # one launch, counted by the kernel itself
    assert relerr(y.cpu().numpy(), refs[0].astype(np.float64) + refs[1]) <= TOL
    ops.clear_caches()


def test_more_tokens_than_the_kernel_holds_use_the_stand_alone_sum(pair):
    from glq_b200 import ops
    rng = np.random.default_rng(9)
    B, m, n = 20, 352, 576
    sh = [_shard(rng, m, n), _shard(rng, m, n)]
    xs = [cuda(rng.standard_normal((B, n)).astype(np.float32), torch.bfloat16) for _ in range(2)]
    refs = [O.linear_forward(xs[r].float().cpu().numpy(), sh[r]["W"], sh[r]["su_h"], sh[r]["sv_h"], sh[r]["ws"]) for r in range(2)]
    call = lambda r: ops.fused_linear_trellis_3inst(xs[r], sh[r]["sv"], sh[r]["su"], sh[r]["p"], None, None, None, None,
                                                    sh[r]["ws"], n, m, n, m, reduce_over=pair[r], out_dtype=torch.float32)
    call(0)
    torch.cuda.synchronize()
    assert pair[0].status(reset=True) == 6
    y = call(1)
    torch.cuda.synchronize()
    assert pair[1].status() == 0
    assert relerr(y.cpu().numpy(), refs[0].astype(np.float64) + refs[1]) <= TOL
    ops.clear_caches()


def test_refused_in_kernel_sum_falls_back_without_rebuilding_plans(pair, monkeypatch):
    """With the single-launch form switched off the plan cannot hold the sum: the operator computes this rank's fp32
    result with the three-launch form and sums it with the stand-alone kernel.  The refusal is remembered, so later
    calls (which may sit inside a CUDA graph capture, where building a plan is not allowed) build nothing."""
    from glq_b200 import ops
    monkeypatch.setenv("GLQB_FUSED_DECODE", "0")
    ops.clear_caches()
    rng = np.random.default_rng(31)
    B, m, n = 2, 352, 576
    sh = [_shard(rng, m, n), _shard(rng, m, n)]
    xs = [cuda(rng.standard_normal((B, n)).astype(np.float32), torch.bfloat16) for _ in range(2)]
    refs = [O.linear_forward(xs[r].float().cpu().numpy(), sh[r]["W"], sh[r]["su_h"], sh[r]["sv_h"], sh[r]["ws"]) for r in range(2)]
    call = lambda r: ops.fused_linear_trellis_3inst(xs[r], sh[r]["sv"], sh[r]["su"], sh[r]["p"], None, None, None, None,
                                                    sh[r]["ws"], n, m, n, m, reduce_over=pair[r], out_dtype=torch.float32)
    call(0)
    torch.cuda.synchronize()
    assert pair[0].status(reset=True) == 6
    y = call(1)
    torch.cuda.synchronize()
    assert pair[1].status() == 0
    assert relerr(y.cpu().numpy(), refs[0].astype(np.float64) + refs[1]) <= TOL
    assert len(ops._REFUSED) == 2                             # one refused form per rank's layer
    plans = len(ops._PLAN_CACHE)
    call(0)                                                   # (gives up again: nobody answers)
    torch.cuda.synchronize()
    assert pair[0].status(reset=True) == 6
    assert len(ops._PLAN_CACHE) == plans and len(ops._REFUSED) == 2
    ops.clear_caches()
