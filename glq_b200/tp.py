"""Tensor-parallel layout of GLQ linears over the GPUs of one node.

The reference has no tensor parallelism of its own: its vLLM loader copies the full tensors to
every rank (glq_vllm/linear_method.py:187-231).  A GLQ matrix cannot be sliced after quantisation,
because the Hadamard transforms mix all rows (SU side) and all columns (SV side); what can be
sharded is the *layer*: each shard is quantised as a GLQ layer of its own, with its own sign vectors
and block decomposition — exactly how the reference already treats the q/k/v and gate/up shards of
a fused projection on one rank (glq_vllm/linear_method.py:825-826, 902-909).

  column-parallel (q, k, v, gate, up): rank r owns output rows [r*m/G, (r+1)*m/G); the input is
      replicated; no exchange.
  row-parallel (o, down): rank r owns input columns [r*n/G, (r+1)*n/G) and produces a full-length
      partial output; the partial outputs are summed over ranks (one all-reduce).

This module only does bookkeeping (shapes, offsets into the flat activation / result buffers, which
result range has to be summed); it runs on CPU tensors as well, which is how the multi-rank logic
is tested (gloo, world size 2).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch

COLUMN_PARALLEL = ("q", "k", "v", "gate", "up")
ROW_PARALLEL = ("o", "down")


@dataclass(frozen=True)
class ShardEntry:
    layer: int
    name: str
    m: int            # rows of this rank's shard
    n: int            # columns of this rank's shard
    x_offset: int     # element offset of the shard's input inside the flat activation buffer
    y_offset: int     # element offset of the shard's output inside the flat result buffer
    row_parallel: bool


@dataclass(frozen=True)
class ShardLayout:
    world: int
    rank: int
    entries: tuple
    x_elems: int
    y_elems: int
    reduce_begin: int     # [reduce_begin, y_elems) holds the row-parallel outputs: summed over ranks


def shard_shape(name: str, m: int, n: int, world: int, row_multiple: int = 32, col_multiple: int = 32):
    """Shape of one rank's shard; refuses splits the kernels cannot read (trellis needs whole 32x32
    groups, E8 whole 8-column index blocks — pass col_multiple=8)."""
    if world == 1:
        return m, n
    if name in COLUMN_PARALLEL:
        if m % world or (m // world) % row_multiple:
            raise ValueError(f"{name}: {m} rows do not split into {world} shards of a multiple of {row_multiple}")
        return m // world, n
    if name in ROW_PARALLEL:
        if n % world or (n // world) % col_multiple:
            raise ValueError(f"{name}: {n} columns do not split into {world} shards of a multiple of {col_multiple}")
        return m, n // world
    raise ValueError(f"unknown projection {name!r}")


def build_layout(proj: Sequence[tuple], n_layers: int, world: int, rank: int,
                 row_multiple: int = 32, col_multiple: int = 32) -> ShardLayout:
    """Flat buffers for a sweep over ``n_layers`` x ``proj`` [(name, m, n), ...]: all column-parallel
    outputs first, then all row-parallel outputs, so that ONE all-reduce covers every partial sum."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    shapes = []
    for li in range(n_layers):
        for name, m, n in proj:
            ms, ns = shard_shape(name, m, n, world, row_multiple, col_multiple)
            shapes.append((li, name, ms, ns, name in ROW_PARALLEL))
    col_total = sum(ms for (_, _, ms, _, rp) in shapes if not rp)
    entries, x_off, y_col, y_row = [], 0, 0, col_total
    for li, name, ms, ns, rp in shapes:
        if rp:
            entries.append(ShardEntry(li, name, ms, ns, x_off, y_row, True))
            y_row += ms
        else:
            entries.append(ShardEntry(li, name, ms, ns, x_off, y_col, False))
            y_col += ms
        x_off += ns
    return ShardLayout(world, rank, tuple(entries), x_off, y_row, col_total)


def all_reduce_row_parallel(y: torch.Tensor, layout: ShardLayout, group=None) -> None:
    """Sum the row-parallel partial outputs over the ranks, in place (NCCL on GPUs, gloo on CPU)."""
    if layout.world == 1 or layout.reduce_begin == layout.y_elems:
        return
    import torch.distributed as dist
    dist.all_reduce(y[layout.reduce_begin:layout.y_elems], op=dist.ReduceOp.SUM, group=group)


# ---------------------------------------------------------------------------------------------------
# Expert parallelism for the MoE grouped matmul: rank r holds experts [r*E/G, (r+1)*E/G), tokens and routing
# are replicated, every rank computes the weighted contributions of ITS experts for all tokens, and one
# all-reduce (sum) of the (tokens, hidden) outputs combines them.  The reference has no multi-GPU MoE; the
# sharding is the usual expert-parallel layout of its host framework.
# ---------------------------------------------------------------------------------------------------
def expert_range(num_experts: int, world: int, rank: int) -> tuple[int, int]:
    """Half-open range of global expert ids owned by ``rank`` (experts must divide evenly)."""
    if num_experts % world:
        raise ValueError(f"{num_experts} experts do not divide over {world} ranks")
    per = num_experts // world
    return rank * per, (rank + 1) * per


def localize_topk_ids(topk_ids: torch.Tensor, e0: int, e1: int) -> torch.Tensor:
    """Global expert ids -> ids local to the rank owning [e0, e1); routings to other ranks' experts become -1,
    which the grouped matmul skips (their weighted contribution is added by the owning rank)."""
    local = topk_ids - e0
    return torch.where((topk_ids >= e0) & (topk_ids < e1), local, torch.full_like(local, -1))


def moe_expert_parallel(run_local, x: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor,
                        num_experts: int, group=None, comm=None) -> torch.Tensor:
    """``run_local(x, local_ids, topk_weights) -> (tokens, hidden)`` computes this rank's experts; the result is
    summed over ranks.  With one rank this is just ``run_local``.  ``comm`` (a ``glq_b200.comm.Comm`` over the same
    ranks): fp32 results that fit its receive area are summed by the library's own one-launch kernel instead of
    NCCL."""
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
    rank = dist.get_rank(group) if world > 1 else 0
    e0, e1 = expert_range(num_experts, world, rank)
    y = run_local(x, localize_topk_ids(topk_ids, e0, e1), topk_weights)
    if world > 1:
        # (one-shot sums send every value to every peer: beyond about a megabyte NCCL's ring / in-switch sums win;
        # measured at 8 GPUs: 0.6 MB 5 % faster than NCCL, 2 MB 6 % slower)
        if (comm is not None and y.dtype == torch.float32 and y.is_contiguous()
                and y.numel() <= min(comm.max_floats, 1 << 18)):
            comm.all_reduce_(y)
        else:
            dist.all_reduce(y, group=group)
    return y
