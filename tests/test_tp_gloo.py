"""Tensor-parallel bookkeeping on CPU ranks (gloo, world size 2): shard shapes, buffer layout, and
that summing row-parallel partial outputs over ranks reproduces the unsharded product."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from glq_b200 import tp
from oracle import glq_oracle as O

PROJ = [("q", 128, 128), ("k", 64, 128), ("v", 64, 128), ("o", 128, 128), ("gate", 192, 128), ("up", 192, 128),
        ("down", 128, 192)]


def test_shard_shapes_and_refusals():
    assert tp.shard_shape("q", 2048, 2048, 8) == (256, 2048)
    assert tp.shard_shape("down", 2048, 11008, 8) == (2048, 1376)
    assert tp.shard_shape("k", 512, 2048, 8) == (64, 2048)
    with pytest.raises(ValueError):
        tp.shard_shape("k", 512, 2048, 32)            # 16 rows per shard: not a whole group
    with pytest.raises(ValueError):
        tp.shard_shape("down", 2048, 11008, 16)       # 688 columns: not a multiple of 32
    assert tp.shard_shape("down", 4096, 14336, 8, col_multiple=8) == (4096, 1792)


def test_layout_is_contiguous_and_reduce_range_is_the_tail():
    lay = tp.build_layout(PROJ, 3, 2, 1)
    assert lay.x_elems == sum(e.n for e in lay.entries)
    assert lay.y_elems == sum(e.m for e in lay.entries)
    col = [e for e in lay.entries if not e.row_parallel]
    row = [e for e in lay.entries if e.row_parallel]
    assert lay.reduce_begin == sum(e.m for e in col)
    spans = sorted((e.y_offset, e.y_offset + e.m) for e in lay.entries)
    assert spans[0][0] == 0 and all(a[1] == b[0] for a, b in zip(spans, spans[1:])) and spans[-1][1] == lay.y_elems
    assert all(e.y_offset >= lay.reduce_begin for e in row) and all(e.y_offset < lay.reduce_begin for e in col)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lay = tp.build_layout(PROJ, 2, world, rank)
        rng = np.random.default_rng(5)                      # same stream on both ranks: full weights / inputs
        y = torch.zeros(lay.y_elems, dtype=torch.float32)
        full = {}
        for li in range(2):
            for name, m, n in PROJ:
                W = rng.standard_normal((m, n)).astype(np.float32)
                x = rng.standard_normal(n).astype(np.float32)
                full[(li, name)] = (W, x)
        for e in lay.entries:
            W, x = full[(e.layer, e.name)]
            if e.row_parallel:          # columns [rank*n_s, (rank+1)*n_s) of W and of x
                Ws, xs = W[:, rank * e.n:(rank + 1) * e.n], x[rank * e.n:(rank + 1) * e.n]
            else:
                Ws, xs = W[rank * e.m:(rank + 1) * e.m], x
            # every shard is a layer of its own: its own signs and Hadamard blocks (identity weights
            # in the rotated domain would hide mistakes, so rotate properly)
            su = (rng.integers(0, 2, size=e.m) * 2 - 1).astype(np.float32)
            sv = (rng.integers(0, 2, size=e.n) * 2 - 1).astype(np.float32)
            bn, bm = O.block_decompose(e.n), O.block_decompose(e.m)
            W_rot = O.block_diag_fht((O.block_diag_fht(Ws * sv[None, :], bn)).T * su[None, :], bm).T
            ys = O.linear_forward(xs[None, :], W_rot, su, sv, 1.0, bn, bm)[0]
            y[e.y_offset:e.y_offset + e.m] = torch.from_numpy(ys)
        tp.all_reduce_row_parallel(y, lay)
        ok = True
        for e in lay.entries:
            W, x = full[(e.layer, e.name)]
            ref = W @ x
            got = y[e.y_offset:e.y_offset + e.m].numpy()
            want = ref if e.row_parallel else ref[rank * e.m:(rank + 1) * e.m]
            ok &= bool(np.allclose(got, want, rtol=1e-4, atol=1e-3))
        out[rank] = ok
    finally:
        dist.destroy_process_group()


def test_two_rank_sweep_matches_unsharded_product():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    out = mgr.dict()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert out.get(0) is True and out.get(1) is True


# ---- expert parallelism of the MoE grouped matmul -----------------------------------------------------------
def test_expert_range_and_id_localisation():
    assert tp.expert_range(128, 8, 3) == (48, 64)
    with pytest.raises(ValueError):
        tp.expert_range(10, 4, 0)
    ids = torch.tensor([[0, 5, 9], [4, 3, 8]])
    loc = tp.localize_topk_ids(ids, 4, 8)
    assert loc.tolist() == [[-1, 1, -1], [0, -1, -1]]


def _moe_dense(x, ids, w, W13, W2, inter):
    """Plain fp32 MoE over the experts in W13/W2 (ids index them; negative ids are skipped)."""
    f13 = lambda e, xb: xb @ W13[e].T
    f2 = lambda e, hb: hb @ W2[e].T
    ids = np.asarray(ids)
    keep = ids >= 0
    wm = np.where(keep, np.asarray(w, np.float32), 0.0).astype(np.float32)
    safe = np.where(keep, ids, ids.max() if keep.any() else 0)          # masked routings get weight 0
    return O.moe_forward(x, safe, wm, f13, f2, inter, "gelu_tanh")


def _moe_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        E, H, I, T, k = 8, 32, 16, 11, 3
        rng = np.random.default_rng(11)                       # same stream on both ranks
        W13 = rng.standard_normal((E, 2 * I, H)).astype(np.float32) * 0.2
        W2 = rng.standard_normal((E, H, I)).astype(np.float32) * 0.2
        x = rng.standard_normal((T, H)).astype(np.float32)
        ids = np.stack([rng.permutation(E)[:k] for _ in range(T)]).astype(np.int64)
        w = rng.random((T, k)).astype(np.float32)
        e0, e1 = tp.expert_range(E, world, rank)

        def run_local(xt, local_ids, wt):
            y = _moe_dense(xt.numpy(), local_ids.numpy(), wt.numpy(), W13[e0:e1], W2[e0:e1], I)
            return torch.from_numpy(y)

        y = tp.moe_expert_parallel(run_local, torch.from_numpy(x), torch.from_numpy(ids), torch.from_numpy(w), E)
        ref = _moe_dense(x, ids, w, W13, W2, I)
        out[rank] = bool(np.allclose(y.numpy(), ref, rtol=1e-5, atol=1e-5))
    finally:
        dist.destroy_process_group()


def test_two_rank_expert_parallel_moe_matches_unsharded():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    out = mgr.dict()
    procs = [ctx.Process(target=_moe_worker, args=(r, world, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert out.get(0) is True and out.get(1) is True
