"""The reference's operator surface for the compressed-weight matmul, served by libglq_b200.

Every function here has the name, positional argument order and return convention of the op the
reference registers under ``torch.ops.glq`` / exposes on its extension module
(glq_vllm/custom_ops.py:39-428, glq/csrc/glq_bindings.cpp:334-550), so the reference's callers
(``E8RHTLinear.forward``, ``_trellis_linear_apply``, ``glq_vllm.linear_method``) work unchanged
when this module is installed in place of the reference extension (see ``glq_b200.dropin``).

Differences, all supersets: activations may be fp16, bf16 or fp32 (the reference casts to fp16
first, glq/quantized_linear.py:1081) and the result comes back in the activation dtype; token
counts above 64 take the tensor-core (tcgen05) GEMM path.
There is no CPU or PyTorch fallback: without a CUDA device and the built library these raise.
"""
from __future__ import annotations

import ctypes as C
import os
from collections import OrderedDict
from typing import Optional, Sequence

import torch

from . import _lib
from .plan import LinearSpec, Plan, block_decompose

DECODE_MAX_TOKENS = 64
# Plans are cheap (a small device table each); what costs memory is the workspace, and that is shared: one
# buffer per (device, stream), grown to the largest plan that ran there.  The cache is least-recently-used
# and bounded; token counts are rounded up to a few bucket sizes so that varying prompt lengths cannot
# create an unbounded number of plans per layer.
PLAN_CACHE_MAX = int(os.environ.get("GLQB_PLAN_CACHE_MAX", "16384"))
_PLAN_CACHE: "OrderedDict" = OrderedDict()
_REFUSED: dict = {}                  # plan keys the library refused (form not available), with the message
_TABLE_CACHE: dict = {}
_WORKSPACES: dict = {}
_RETIRED_WORKSPACES: list = []      # outgrown buffers stay alive: captured CUDA graphs may still point at them
_META_CACHE: dict = {}


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"glq_b200: {name} must be a CUDA tensor (there is no CPU path)")


def _blocks(t, fallback: int) -> list[int]:
    if t is None:
        return block_decompose(fallback)
    if isinstance(t, torch.Tensor):
        if t.numel() == 0:
            return block_decompose(fallback)
        return [int(v) for v in t.tolist()]
    return [int(v) for v in t]


def e8_packed_table(codebook: torch.Tensor) -> torch.Tensor:
    """fp16 (entries, 8) codebook -> cached nibble-packed int32 (entries,) table on its device."""
    _require_cuda(codebook, "codebook")
    key = (codebook.data_ptr(), codebook.shape[0], codebook.device.index, codebook.dtype)
    tb = _TABLE_CACHE.get(key)
    if tb is None:
        cb = codebook.to(torch.float16).contiguous()
        tb = torch.empty(cb.shape[0], dtype=torch.int32, device=cb.device)
        _lib.check(_lib.load().glqb_e8_pack_table(cb.data_ptr(), cb.shape[0], tb.data_ptr(), _stream(cb)),
                   "e8_pack_table")
        # the key is an address: keep the source alive so the address cannot be handed to another tensor
        _TABLE_CACHE[key] = (tb, codebook)
        return tb
    return tb[0]


def token_bucket(b: int) -> int:
    """Token count a plan is built for when ``b`` tokens arrive: exact up to 8, multiples of 8 up to 64
    (the streaming kernels), 128, then multiples of 256 (the tensor-core path).  Inputs are zero-padded to
    the bucket and the extra output rows dropped."""
    if b <= 8:
        return b
    if b <= DECODE_MAX_TOKENS:
        return (b + 7) // 8 * 8
    if b <= 128:
        return 128
    return (b + 255) // 256 * 256


def shared_workspace(device, nbytes: int) -> torch.Tensor:
    """The workspace every cached plan on (device, current stream) runs in; grows geometrically."""
    dev = torch.device(device)
    key = (dev.index if dev.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(dev).cuda_stream)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < nbytes:
        if ws is not None:
            _RETIRED_WORKSPACES.append(ws)
        size = max(nbytes, 2 * ws.numel() if ws is not None else 0, 1 << 20)
        ws = torch.empty(size, dtype=torch.uint8, device=dev)
        _WORKSPACES[key] = ws
    return ws


def _cached_plan(key, make_specs) -> Plan:
    p = _PLAN_CACHE.get(key)
    if p is not None:
        _PLAN_CACHE.move_to_end(key)
        return p
    p = Plan(make_specs(), own_workspace=False)
    _PLAN_CACHE[key] = p
    if len(_PLAN_CACHE) > PLAN_CACHE_MAX and not torch.cuda.is_current_stream_capturing():
        # evict the least recently used plans; their device tables may still be read by queued work
        torch.cuda.synchronize()
        while len(_PLAN_CACHE) > PLAN_CACHE_MAX:
            _, old = _PLAN_CACHE.popitem(last=False)
            old.close()
    return p


def check_device_status() -> None:
    """Synchronise and raise RuntimeError (code GLQB_E_DEVICE) if a kernel of any cached plan gave up on one
    of its bounded waits since the plan was built: the results of that run are invalid.  Cheap enough for
    the points where a caller synchronises anyway (end of a request, a test, a benchmark step)."""
    for p in list(_PLAN_CACHE.values()):
        if hasattr(p, "check_status"):
            p.check_status()


def clear_caches() -> None:
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    for p in _PLAN_CACHE.values():
        p.close()
    _PLAN_CACHE.clear()
    _REFUSED.clear()
    _TABLE_CACHE.clear()
    _WORKSPACES.clear()
    _RETIRED_WORKSPACES.clear()
    _META_CACHE.clear()


def _run_sliced(x2d: torch.Tensor, out: torch.Tensor, key_base, make_spec, max_tokens=DECODE_MAX_TOKENS,
                y_offset: int = 0, out_cols: Optional[int] = None, accumulate: bool = False, comm=None) -> None:
    """Run a single-layer op over x2d (B, in) into out[:, y_offset : y_offset + out_cols].  Up to 64 tokens go
    through the streaming kernels in slices of <= max_tokens, more through one tensor-core plan; token counts
    are rounded up to ``token_bucket`` sizes (zero-padded copy in, extra rows dropped)."""
    B = x2d.shape[0]
    cols = out_cols if out_cols is not None else out.shape[1]

    def run(xs, b, dst_rows):
        bb = token_bucket(b)
        if bb == b:
            xin, yout, yoff = xs, dst_rows, y_offset
        else:
            xin = xs.new_zeros((bb, xs.shape[1]))
            xin[:b] = xs
            yout, yoff = torch.empty((bb, cols), dtype=out.dtype, device=out.device), 0
            if accumulate:
                yout[:b] = dst_rows[:b, y_offset:y_offset + cols]
        key = key_base + (bb, xin.dtype, yout.dtype, xin.stride(0), yout.stride(0), yoff, id(comm) if comm is not None else 0)
        refused = _REFUSED.get(key)
        if refused is not None:                       # the library refused this form before: do not build the plan again
            raise RuntimeError(refused)
        fresh = key not in _PLAN_CACHE
        try:
            plan = _cached_plan(key, lambda: [make_spec(bb, xin.stride(0), yout.stride(0), yoff)])
            if fresh and comm is not None:
                try:
                    plan.set_comm(comm)
                except RuntimeError:
                    _PLAN_CACHE.pop(key).close()
                    raise
        except RuntimeError as e:
            # callers fall back to another form on these two refusals, call after call (also inside graph capture,
            # where building and freeing a plan is not allowed): remember them
            if "single-launch" in str(e) or "plan_set_comm" in str(e):
                _REFUSED[key] = str(e)
            raise
        plan.run(xin, yout, workspace=shared_workspace(xin.device, plan.workspace_bytes))
        if bb != b:
            dst_rows[:b, y_offset:y_offset + cols] = yout[:b]

    if B > DECODE_MAX_TOKENS:
        run(x2d, B, out)
        return
    done = 0
    while done < B:
        b = min(max_tokens, B - done)
        run(x2d[done:done + b], b, out[done:done + b])
        done += b


# ------------------------------------------------------------------------------------------------
# trellis 3INST fused linears (glq_vllm/custom_ops.py:373-418)
# ------------------------------------------------------------------------------------------------
def _trellis_bits(packed: torch.Tensor) -> int:
    return packed.shape[-1] // 16


FUSED_MAX_TOKENS = 8        # the single-launch decode form, which also serves the fused norm / activation / residual


class _InKernel:
    """Marks a communicator whose sum the decode kernel itself performs (internal to _fused_trellis)."""

    def __init__(self, comm):
        self.comm = comm
        self.world = comm.world


def _apply_input_steps(x2d, in_features, in_norm_weight, in_norm_eps, gated_act):
    """The steps the single-launch form fuses, as separate torch kernels (more than 8 tokens)."""
    if gated_act is not None:
        g, u = x2d[:, :in_features], x2d[:, in_features:2 * in_features]
        a = (torch.nn.functional.silu(g) if gated_act == 0 else
             torch.nn.functional.gelu(g, approximate="tanh") if gated_act == 1 else torch.relu(g).square())
        x2d = a * u
    if in_norm_weight is not None:
        xf = x2d.float()
        xn = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + in_norm_eps)).to(x2d.dtype)
        x2d = (in_norm_weight.to(x2d.dtype) * xn)
    return x2d.contiguous()


def _fused_trellis(x, sv, su, packed, packed2, blocks_n, blocks_m, wscale, inv_rs2, in_features,
                   out_features, n_pad, m_pad, y_rht_out=None, col=0, out_dtype=None,
                   in_norm_weight=None, in_norm_eps=1e-6, gated_act=None, accumulate_into=None, reduce_over=None):
    _require_cuda(x, "x")
    comm = None
    if isinstance(reduce_over, _InKernel):
        comm, reduce_over = reduce_over.comm, None
    if reduce_over is not None and reduce_over.world == 1:
        reduce_over = None
    if reduce_over is not None:
        if y_rht_out is not None:
            raise RuntimeError("glq_b200: reduce_over applies to complete linears only")
        ntok = x.reshape(-1, in_features * (2 if gated_act is not None else 1)).shape[0]
        fits = ntok <= FUSED_MAX_TOKENS
        if fits:
            try:
                return _fused_trellis(x, sv, su, packed, packed2, blocks_n, blocks_m, wscale, inv_rs2, in_features,
                                      out_features, n_pad, m_pad, out_dtype=out_dtype, in_norm_weight=in_norm_weight,
                                      in_norm_eps=in_norm_eps, gated_act=gated_act, accumulate_into=accumulate_into,
                                      reduce_over=_InKernel(reduce_over))
            except RuntimeError as e:
                if "plan_set_comm" not in str(e) and "single-launch" not in str(e):
                    raise
        # the kernel cannot hold the sum (more than 8 tokens, or no single-launch form): fp32 partial result, then one
        # launch of the stand-alone sum (or NCCL when it exceeds the communicator's area)
        part = _fused_trellis(x, sv, su, packed, packed2, blocks_n, blocks_m, wscale, inv_rs2, in_features,
                              out_features, n_pad, m_pad, out_dtype=torch.float32, in_norm_weight=in_norm_weight,
                              in_norm_eps=in_norm_eps, gated_act=gated_act)
        if part.numel() <= reduce_over.max_floats:
            reduce_over.all_reduce_(part)
        else:
            import torch.distributed as dist
            dist.all_reduce(part)
        if accumulate_into is not None:
            accumulate_into.add_(part.reshape(accumulate_into.shape).to(accumulate_into.dtype))
            return accumulate_into
        return part.to(out_dtype or x.dtype)
    x_cols = in_features * (2 if gated_act is not None else 1)
    x2d = x.reshape(-1, x_cols)
    if x2d.stride(-1) != 1:
        x2d = x2d.contiguous()
    extras = in_norm_weight is not None or gated_act is not None or accumulate_into is not None
    if extras:
        if y_rht_out is not None:
            raise RuntimeError("glq_b200: fused norm / activation / residual steps apply to complete linears only")
        if x2d.shape[0] > FUSED_MAX_TOKENS:
            # more tokens than the single-launch form takes: run the steps as their own kernels
            xin = _apply_input_steps(x2d, in_features, in_norm_weight, in_norm_eps, gated_act)
            y = _fused_trellis(xin, sv, su, packed, packed2, blocks_n, blocks_m, wscale, inv_rs2, in_features,
                               out_features, n_pad, m_pad, out_dtype=out_dtype)
            if accumulate_into is not None:
                accumulate_into.add_(y.reshape(accumulate_into.shape).to(accumulate_into.dtype))
                return accumulate_into
            return y
    has2 = packed2 is not None and packed2.numel() > 0
    codes = [packed] + ([packed2] if has2 else [])
    bits = [_trellis_bits(packed)] + ([_trellis_bits(packed2)] if has2 else [])
    bn, bm = _blocks(blocks_n, n_pad), _blocks(blocks_m, m_pad)
    if accumulate_into is not None:
        tgt, yoff, stop = accumulate_into.reshape(-1, out_features), 0, False
        if tgt.data_ptr() != accumulate_into.data_ptr() or tgt.stride(-1) != 1:
            raise RuntimeError("glq_b200: accumulate_into must be a dense (tokens, out_features) tensor")
    elif y_rht_out is None:
        out = torch.empty(x2d.shape[0], out_features, dtype=out_dtype or x2d.dtype, device=x2d.device)
        tgt, yoff, stop = out, 0, False
    else:
        tgt, yoff, stop = y_rht_out, int(col), True

    def make_spec(b, x_stride, y_stride, y_offset):
        return LinearSpec(format=_lib.FMT_TRELLIS_3INST, m_pad=m_pad, n_pad=n_pad, in_features=in_features,
                          out_features=out_features if not stop else m_pad, codes=codes, bits=bits, su=su, sv=sv,
                          wscale=float(wscale), stage_scale=[float(inv_rs2)] if has2 else [],
                          blocks_n=bn, blocks_m=bm, batch=b, x_dtype=x2d.dtype, y_dtype=tgt.dtype,
                          x_stride=x_stride, y_stride=y_stride, y_offset=y_offset, stop_at_yrht=stop,
                          in_norm_weight=in_norm_weight, in_norm_eps=in_norm_eps, in_gated_act=gated_act,
                          y_accumulate=accumulate_into is not None)

    key = ("trellis", packed.data_ptr(), packed2.data_ptr() if has2 else 0, su.data_ptr() if su is not None else 0,
           sv.data_ptr(), float(wscale), float(inv_rs2), m_pad, n_pad, out_features, stop,
           in_norm_weight.data_ptr() if in_norm_weight is not None else 0, float(in_norm_eps), gated_act,
           accumulate_into is not None)
    # two decoded stages keep two accumulator sets: 32 tokens per pass instead of 64
    try:
        _run_sliced(x2d, tgt, key, make_spec, 32 if has2 else DECODE_MAX_TOKENS, y_offset=yoff,
                    out_cols=m_pad if stop else out_features, accumulate=accumulate_into is not None, comm=comm)
    except RuntimeError as e:
        if comm is not None or not extras or "single-launch" not in str(e):
            raise
        # the single-launch form is unavailable for this layer (switched off, or the input does not fit in
        # shared memory): run the steps as their own kernels
        xin = _apply_input_steps(x2d, in_features, in_norm_weight, in_norm_eps, gated_act)
        y = _fused_trellis(xin, sv, su, packed, packed2, blocks_n, blocks_m, wscale, inv_rs2, in_features,
                           out_features, n_pad, m_pad, out_dtype=out_dtype)
        if accumulate_into is None:
            return y
        accumulate_into.add_(y.reshape(accumulate_into.shape).to(accumulate_into.dtype))
    if accumulate_into is not None:
        return accumulate_into
    return None if stop else tgt


def fused_linear_trellis_3inst(x, sv, su, trellis_packed, blocks_n, blocks_m, blocks_n_meta, blocks_m_meta,
                               wscale, in_features, out_features, n_pad, m_pad, *, out_dtype=None,
                               in_norm_weight=None, in_norm_eps=1e-6, gated_act=None, accumulate_into=None,
                               reduce_over=None):
    """input RHT -> 3INST decode + matmul -> x Wscale -> output RHT, (B, in) -> (B, out).
    Keyword arguments that are not in the reference: ``out_dtype`` selects the result dtype (default: that of
    x); ``in_norm_weight`` / ``in_norm_eps`` apply an RMSNorm to x first; ``gated_act`` (0 silu, 1 gelu-tanh,
    2 relu^2) takes x as [gate | up] of 2 * in_features values and feeds act(gate) * up; ``accumulate_into``
    adds the result to that (B, out) tensor in place (residual add) and returns it.  Up to 8 tokens these run
    inside the one decode kernel, above that as separate torch kernels around the linear.
    ``reduce_over`` (a ``glq_b200.comm.Comm``): this rank holds a column shard of a row-parallel layer; the result
    (and what is added to ``accumulate_into``) is the sum over the communicator's ranks, formed inside the decode
    kernel up to 8 tokens, else by one extra launch."""
    return _fused_trellis(x, sv, su, trellis_packed, None, blocks_n, blocks_m, wscale, 0.0,
                          in_features, out_features, n_pad, m_pad, out_dtype=out_dtype, in_norm_weight=in_norm_weight,
                          in_norm_eps=in_norm_eps, gated_act=gated_act, accumulate_into=accumulate_into,
                          reduce_over=reduce_over)


def fused_linear_trellis_3inst_rvq2(x, sv, su, trellis_packed, trellis_packed2, blocks_n, blocks_m,
                                    blocks_n_meta, blocks_m_meta, wscale, inv_resid_scale2,
                                    in_features, out_features, n_pad, m_pad, out_dtype=None):
    """Stacked two-stage (5-8 bpw) form: W = dec(stage1) + inv_resid_scale2 * dec(stage2)."""
    return _fused_trellis(x, sv, su, trellis_packed, trellis_packed2, blocks_n, blocks_m, wscale,
                          inv_resid_scale2, in_features, out_features, n_pad, m_pad, out_dtype=out_dtype)


def fused_linear_trellis_3inst_yrht(x, sv, trellis_packed, blocks_n, blocks_n_meta, wscale,
                                    in_features, n_pad, m_pad, y_rht_out, col):
    """Stops before the output transform: deposits fp32 rotated outputs into y_rht_out[:, col:col+m_pad]."""
    dummy_su = _ones_f16(m_pad, x.device)
    _fused_trellis(x, sv, dummy_su, trellis_packed, None, blocks_n, None, wscale, 0.0,
                   in_features, m_pad, n_pad, m_pad, y_rht_out=y_rht_out, col=col)


def fused_linear_trellis_3inst_yrht_rvq2(x, sv, trellis_packed, trellis_packed2, blocks_n, blocks_n_meta,
                                         wscale, inv_resid_scale2, in_features, n_pad, m_pad, y_rht_out, col):
    dummy_su = _ones_f16(m_pad, x.device)
    _fused_trellis(x, sv, dummy_su, trellis_packed, trellis_packed2, blocks_n, None, wscale, inv_resid_scale2,
                   in_features, m_pad, n_pad, m_pad, y_rht_out=y_rht_out, col=col)


def fused_linear_trellis_3inst_shards(x, sv, shards, blocks_n=None, out_dtype=None, in_norm_weight=None, in_norm_eps=1e-6):
    """Several trellis layers that read the same input (the q/k/v or gate/up shards of a fused projection, which
    share SV: glq_vllm/linear_method.py:825-826, 902-909) as ONE plan: one launch for up to 8 tokens instead of
    one fused call per shard plus a shard-batched output transform (glq_vllm/linear_method.py:662-710).
    ``shards`` is a sequence of (su, trellis_packed, trellis_packed2 or None, wscale, inv_resid_scale2, m_pad);
    returns (B, sum of m_pad) with the shards' outputs side by side.  ``in_norm_weight`` applies an RMSNorm to x
    first (inside the kernel up to 8 tokens).  Not in the reference."""
    _require_cuda(x, "x")
    n = sv.numel()
    x2d = x.reshape(-1, n)
    if x2d.stride(-1) != 1:
        x2d = x2d.contiguous()
    B = x2d.shape[0]
    if in_norm_weight is not None and B > FUSED_MAX_TOKENS:
        x2d, in_norm_weight = _apply_input_steps(x2d, n, in_norm_weight, in_norm_eps, None), None
    total_m = sum(int(sh[5]) for sh in shards)
    odt = out_dtype or x2d.dtype
    bn = _blocks(blocks_n, n)
    bb = token_bucket(B)
    xin = x2d
    if bb != B:
        xin = x2d.new_zeros((bb, n))
        xin[:B] = x2d
    out = torch.empty((bb, total_m), dtype=odt, device=x2d.device)
    key = ("trellis_shards", tuple(sh[1].data_ptr() for sh in shards), sv.data_ptr(), tuple(float(sh[3]) for sh in shards),
           bb, xin.dtype, odt, xin.stride(0), in_norm_weight.data_ptr() if in_norm_weight is not None else 0, float(in_norm_eps))

    def make_specs():
        specs, col = [], 0
        for su, packed, packed2, wscale, inv2, m in shards:
            has2 = packed2 is not None and packed2.numel() > 0
            specs.append(LinearSpec(format=_lib.FMT_TRELLIS_3INST, m_pad=int(m), n_pad=n, in_features=n, out_features=int(m),
                                    codes=[packed] + ([packed2] if has2 else []),
                                    bits=[_trellis_bits(packed)] + ([_trellis_bits(packed2)] if has2 else []),
                                    su=su, sv=sv, wscale=float(wscale), stage_scale=[float(inv2)] if has2 else [],
                                    blocks_n=bn, blocks_m=block_decompose(int(m)), batch=bb, x_dtype=xin.dtype, y_dtype=odt,
                                    x_stride=xin.stride(0), y_stride=total_m, y_offset=col,
                                    in_norm_weight=in_norm_weight, in_norm_eps=in_norm_eps))
            col += int(m)
        return specs
    plan = _cached_plan(key, make_specs)
    plan.run(xin, out, workspace=shared_workspace(xin.device, plan.workspace_bytes))
    return out[:B]


def fused_linear_e8_shards(x, sv, shards, codebook, codebook2=None, blocks_n=None, out_dtype=None, in_norm_weight=None,
                           in_norm_eps=1e-6):
    """Several unpadded (block-diagonal) E8-shell layers that read the same input — the q/k/v or gate/up parts of a
    merged layer whose parts share SV — as ONE plan: one launch for up to 8 tokens.  ``shards`` is a sequence of
    (su, [qidxs, qidxs2, ...], [inv_resid_scale, ...], wscale, m_pad); ``codebook`` the fp16 (65536, 8) table,
    ``codebook2`` the table of the second stage when it differs (the 256-entry one).  Returns (B, sum of m_pad).
    ``in_norm_weight`` applies an RMSNorm to x first.  Not in the reference."""
    _require_cuda(x, "x")
    n = sv.numel()
    x2d = x.reshape(-1, n)
    if x2d.stride(-1) != 1:
        x2d = x2d.contiguous()
    B = x2d.shape[0]
    if in_norm_weight is not None and B > FUSED_MAX_TOKENS:
        x2d, in_norm_weight = _apply_input_steps(x2d, n, in_norm_weight, in_norm_eps, None), None
    total_m = sum(int(sh[4]) for sh in shards)
    odt = out_dtype or x2d.dtype
    bn = _blocks(blocks_n, n)
    bb = token_bucket(B)
    xin = x2d
    if bb != B:
        xin = x2d.new_zeros((bb, n))
        xin[:B] = x2d
    out = torch.empty((bb, total_m), dtype=odt, device=x2d.device)
    t1 = e8_packed_table(codebook)
    t2 = e8_packed_table(codebook2) if codebook2 is not None else t1
    key = ("e8_shards", tuple(sh[1][0].data_ptr() for sh in shards), sv.data_ptr(), tuple(float(sh[3]) for sh in shards),
           t1.data_ptr(), t2.data_ptr(), bb, xin.dtype, odt, xin.stride(0),
           in_norm_weight.data_ptr() if in_norm_weight is not None else 0, float(in_norm_eps))

    def make_specs():
        specs, col = [], 0
        for su, qs, inv, wscale, m in shards:
            tables = [t1] + [t2 if k == 1 else t1 for k in range(1, len(qs))]
            specs.append(LinearSpec(format=_lib.FMT_E8_SHELL, m_pad=int(m), n_pad=n, in_features=n, out_features=int(m),
                                    codes=list(qs), tables=tables, stage_scale=[float(v) for v in inv], su=su, sv=sv,
                                    wscale=float(wscale), blocks_n=bn, blocks_m=block_decompose(int(m)), batch=bb,
                                    x_dtype=xin.dtype, y_dtype=odt, x_stride=xin.stride(0), y_stride=total_m, y_offset=col,
                                    in_norm_weight=in_norm_weight, in_norm_eps=in_norm_eps))
            col += int(m)
        return specs
    plan = _cached_plan(key, make_specs)
    plan.run(xin, out, workspace=shared_workspace(xin.device, plan.workspace_bytes))
    return out[:B]


_ONES: dict = {}


def _ones_f16(n: int, device) -> torch.Tensor:
    key = (n, str(device))
    t = _ONES.get(key)
    if t is None:
        t = torch.ones(n, dtype=torch.float16, device=device)
        _ONES[key] = t
    return t


def output_rht_shards(y_rht, su, y, out_features, shard_meta, max_bs):
    """One output transform over the sub-blocks of several shards (glq_vllm/custom_ops.py:424-426).
    shard_meta rows are (global column offset, block size, log2, optional normalisation bits); the offsets are
    honoured.  The reference keeps the meta on the device; its host copy is read once per tensor (the first
    call, which therefore has to happen outside stream capture, like the reference's own warm-up) and cached."""
    _require_cuda(y_rht, "y_rht")
    if isinstance(shard_meta, torch.Tensor):
        key = (shard_meta.data_ptr(), shard_meta.numel(), str(shard_meta.device))
        hit = _META_CACHE.get(key)
        if hit is None:
            hit = (shard_meta.cpu().tolist(), shard_meta)       # keeps the tensor (and its address) alive
            _META_CACHE[key] = hit
        meta = hit[0]
    else:
        meta = list(shard_meta)
    offsets = [int(r[0]) for r in meta]
    blocks = [int(r[1]) for r in meta]
    B = y_rht.shape[0]
    lib = _lib.load()
    # at most MAX_BLOCKS sub-blocks per launch
    for i in range(0, len(blocks), _lib.MAX_BLOCKS):
        o, b = offsets[i:i + _lib.MAX_BLOCKS], blocks[i:i + _lib.MAX_BLOCKS]
        _lib.check(lib.glqb_output_rht_shards(y_rht.data_ptr(), su.data_ptr(), y.data_ptr(), _dt(y.dtype), y.stride(0),
                                              int(out_features), int(y_rht.shape[1]), (C.c_int32 * len(o))(*o),
                                              (C.c_int32 * len(b))(*b), len(b), B, _stream(y)), "output_rht_shards")


def _dt(dtype) -> int:
    return {torch.float16: _lib.DT_F16, torch.bfloat16: _lib.DT_BF16, torch.float32: _lib.DT_F32}[dtype]


# ------------------------------------------------------------------------------------------------
# E8 shell fused linears (glq_vllm/custom_ops.py:105-126)
# ------------------------------------------------------------------------------------------------
def _e8_stages(qidxs, codebook, qidxs2, codebook2, inv_rs, qidxs3, codebook3, inv_rs2, qidxs4, codebook4, inv_rs3):
    codes, tables, scales = [qidxs], [e8_packed_table(codebook)], []
    for q, cb, s in ((qidxs2, codebook2, inv_rs), (qidxs3, codebook3, inv_rs2), (qidxs4, codebook4, inv_rs3)):
        if q is None or q.numel() == 0 or cb is None or cb.numel() == 0 or float(s) == 0.0:
            break
        codes.append(q)
        tables.append(e8_packed_table(cb))
        scales.append(float(s))
    return codes, tables, scales


def _fused_e8(x, sv, su, codes, tables, scales, wscale, in_features, out_features, n_pad, m_pad, bn, bm,
              x_is_rotated=False, stop=False, out_dtype=None, in_norm_weight=None, in_norm_eps=1e-6, gated_act=None,
              accumulate_into=None, reduce_over=None, _in_kernel=False):
    _require_cuda(x, "x")
    comm = reduce_over if (reduce_over is not None and reduce_over.world > 1) else None
    extras = in_norm_weight is not None or gated_act is not None or accumulate_into is not None
    if (extras or comm is not None) and not _in_kernel:
        if stop or x_is_rotated:
            raise RuntimeError("glq_b200: fused norm / activation / residual / rank-sum steps apply to complete linears only")
        x2 = x.reshape(-1, in_features * (2 if gated_act is not None else 1))
        args = (sv, su, codes, tables, scales, wscale, in_features, out_features, n_pad, m_pad, bn, bm)
        if x2.shape[0] <= FUSED_MAX_TOKENS:
            try:                                             # all steps inside the one decode kernel
                return _fused_e8(x2, *args, out_dtype=out_dtype, in_norm_weight=in_norm_weight, in_norm_eps=in_norm_eps,
                                 gated_act=gated_act, accumulate_into=accumulate_into, reduce_over=comm, _in_kernel=True)
            except RuntimeError as e:
                if "single-launch" not in str(e) and "plan_set_comm" not in str(e):
                    raise
        # more than 8 tokens, or no single-launch form for this layer: the steps as kernels of their own
        xin = _apply_input_steps(x2, in_features, in_norm_weight, in_norm_eps, gated_act)
        y = _fused_e8(xin, *args, out_dtype=torch.float32 if comm is not None else out_dtype)
        if comm is not None:
            if y.numel() <= comm.max_floats:
                comm.all_reduce_(y)
            else:
                import torch.distributed as dist
                dist.all_reduce(y)
        if accumulate_into is not None:
            accumulate_into.add_(y.reshape(accumulate_into.shape).to(accumulate_into.dtype))
            return accumulate_into
        return y if comm is None else y.to(out_dtype or x.dtype)
    feat_in = n_pad if x_is_rotated else in_features
    x2d = x.reshape(-1, feat_in * (2 if gated_act is not None else 1))
    if x2d.stride(-1) != 1:
        x2d = x2d.contiguous()
    odt = torch.float32 if stop else (out_dtype or x2d.dtype)
    if accumulate_into is not None:
        out = accumulate_into.reshape(-1, out_features)
        if out.data_ptr() != accumulate_into.data_ptr() or out.stride(-1) != 1:
            raise RuntimeError("glq_b200: accumulate_into must be a dense (tokens, out_features) tensor")
        odt = out.dtype
    else:
        out = torch.empty(x2d.shape[0], m_pad if stop else out_features, dtype=odt, device=x2d.device)

    def make_spec(b, x_stride, y_stride, y_offset):
        return LinearSpec(format=_lib.FMT_E8_SHELL, m_pad=m_pad, n_pad=n_pad, in_features=feat_in,
                          out_features=m_pad if stop else out_features, codes=codes, tables=tables,
                          stage_scale=scales, su=su, sv=sv, wscale=float(wscale), blocks_n=bn, blocks_m=bm,
                          batch=b, x_dtype=x2d.dtype, y_dtype=odt, x_stride=x_stride, y_stride=y_stride,
                          y_offset=y_offset, stop_at_yrht=stop, x_is_rotated=x_is_rotated,
                          in_norm_weight=in_norm_weight, in_norm_eps=in_norm_eps, in_gated_act=gated_act,
                          y_accumulate=accumulate_into is not None)

    key = ("e8", tuple(c.data_ptr() for c in codes), tuple(t.data_ptr() for t in tables), tuple(scales),
           su.data_ptr(), sv.data_ptr(), float(wscale), m_pad, n_pad, in_features, out_features, stop, x_is_rotated,
           in_norm_weight.data_ptr() if in_norm_weight is not None else 0, float(in_norm_eps), gated_act,
           accumulate_into is not None)
    _run_sliced(x2d, out, key, make_spec, 32 if len(codes) > 2 else DECODE_MAX_TOKENS,
                accumulate=accumulate_into is not None, comm=comm)
    return accumulate_into if accumulate_into is not None else out


_EMPTY = None


def fused_linear(x, sv, su, qidxs, codebook, wscale, in_features, out_features, n_pad, m_pad, log_n, log_m,
                 qidxs2=_EMPTY, codebook2=_EMPTY, inv_resid_scale=0.0, qidxs3=_EMPTY, codebook3=_EMPTY,
                 inv_resid_scale2=0.0, qidxs4=_EMPTY, codebook4=_EMPTY, inv_resid_scale3=0.0, out_dtype=None, *,
                 in_norm_weight=None, in_norm_eps=1e-6, gated_act=None, accumulate_into=None, reduce_over=None):
    """Power-of-two padded E8 layer: whole-length Hadamard on both sides.  The keyword-only arguments are those of
    ``fused_linear_trellis_3inst`` (not in the reference)."""
    codes, tables, scales = _e8_stages(qidxs, codebook, qidxs2, codebook2, inv_resid_scale, qidxs3, codebook3,
                                       inv_resid_scale2, qidxs4, codebook4, inv_resid_scale3)
    return _fused_e8(x, sv, su, codes, tables, scales, wscale, in_features, out_features, n_pad, m_pad,
                     [n_pad], [m_pad], out_dtype=out_dtype, in_norm_weight=in_norm_weight, in_norm_eps=in_norm_eps,
                     gated_act=gated_act, accumulate_into=accumulate_into, reduce_over=reduce_over)


def fused_linear_block_diag(x, sv, su, qidxs, codebook, wscale, in_features, out_features, n_pad, m_pad,
                            blocks_n, blocks_m, blocks_n_meta, blocks_m_meta,
                            qidxs2=_EMPTY, codebook2=_EMPTY, inv_resid_scale=0.0, qidxs3=_EMPTY, codebook3=_EMPTY,
                            inv_resid_scale2=0.0, qidxs4=_EMPTY, codebook4=_EMPTY, inv_resid_scale3=0.0,
                            out_dtype=None, *, in_norm_weight=None, in_norm_eps=1e-6, gated_act=None,
                            accumulate_into=None, reduce_over=None):
    """Unpadded E8 layer with block-diagonal Hadamards.  Keyword-only arguments that are not in the reference, as
    on ``fused_linear_trellis_3inst``: ``in_norm_weight`` / ``in_norm_eps`` (RMSNorm in front), ``gated_act``
    (x holds [gate | up]), ``accumulate_into`` (residual add), ``reduce_over`` (sum over tensor-parallel ranks);
    up to 8 tokens they run inside the one decode kernel."""
    codes, tables, scales = _e8_stages(qidxs, codebook, qidxs2, codebook2, inv_resid_scale, qidxs3, codebook3,
                                       inv_resid_scale2, qidxs4, codebook4, inv_resid_scale3)
    return _fused_e8(x, sv, su, codes, tables, scales, wscale, in_features, out_features, n_pad, m_pad,
                     _blocks(blocks_n, n_pad), _blocks(blocks_m, m_pad), out_dtype=out_dtype,
                     in_norm_weight=in_norm_weight, in_norm_eps=in_norm_eps, gated_act=gated_act,
                     accumulate_into=accumulate_into, reduce_over=reduce_over)


def dequant_matmul(x, qidxs, codebook, wscale, qidxs2=_EMPTY, codebook2=_EMPTY, inv_resid_scale=0.0,
                   codebook_abs=None, qidxs3=_EMPTY, codebook3=_EMPTY, inv_resid_scale2=0.0,
                   qidxs4=_EMPTY, codebook4=_EMPTY, inv_resid_scale3=0.0):
    """Rotated-domain product only: x (B, n_pad) already transformed -> fp32 (B, m_pad) scaled by wscale."""
    m_pad, n_pad = qidxs.shape[0], qidxs.shape[1] * 8
    codes, tables, scales = _e8_stages(qidxs, codebook, qidxs2, codebook2, inv_resid_scale, qidxs3, codebook3,
                                       inv_resid_scale2, qidxs4, codebook4, inv_resid_scale3)
    ones_m, ones_n = _ones_f16(m_pad, x.device), _ones_f16(n_pad, x.device)
    return _fused_e8(x, ones_n, ones_m, codes, tables, scales, wscale, n_pad, m_pad, n_pad, m_pad,
                     block_decompose(n_pad), block_decompose(m_pad), x_is_rotated=True, stop=True)


def dequant_matvec(x, qidxs, codebook, wscale, qidxs2=_EMPTY, codebook2=_EMPTY, inv_resid_scale=0.0,
                   codebook_abs=None):
    """(n_pad,) rotated activations -> fp32 (m_pad,)."""
    return dequant_matmul(x.reshape(1, -1), qidxs, codebook, wscale, qidxs2, codebook2, inv_resid_scale).reshape(-1)


def input_rht(x, sv, out, in_features, stride_x, rsqrt_n, n_pad, log_n):
    """out (B, n_pad) fp32 <- H(SV * pad(x)) / sqrt(n_pad), whole-length transform."""
    _require_cuda(x, "x")
    B = out.shape[0]
    arr = (C.c_int32 * 1)(int(n_pad))
    _lib.check(_lib.load().glqb_input_rht(x.data_ptr(), _dt(x.dtype), int(stride_x), sv.data_ptr(), out.data_ptr(),
                                          int(in_features), int(n_pad), arr, 1, B, _stream(x)), "input_rht")


def input_rht_blocks(x, sv, out, in_features, n_pad, blocks):
    """Block-diagonal form of :func:`input_rht`."""
    B = out.shape[0]
    bl = _blocks(blocks, n_pad)
    arr = (C.c_int32 * len(bl))(*bl)
    _lib.check(_lib.load().glqb_input_rht(x.data_ptr(), _dt(x.dtype), x.stride(0), sv.data_ptr(), out.data_ptr(),
                                          int(in_features), int(n_pad), arr, len(bl), B, _stream(x)), "input_rht")


def output_rht(y_rht, su, out, out_features, m_pad, log_m, rsqrt_m):
    """out (B, out_features) <- (SU * H(y_rht) / sqrt(m_pad))[:, :out_features]."""
    _require_cuda(y_rht, "y_rht")
    B = y_rht.shape[0]
    arr = (C.c_int32 * 1)(int(m_pad))
    _lib.check(_lib.load().glqb_output_rht(y_rht.data_ptr(), su.data_ptr(), out.data_ptr(), _dt(out.dtype),
                                           out.stride(0), int(out_features), int(m_pad), arr, 1, B, _stream(out)),
               "output_rht")


def output_rht_blocks(y_rht, su, out, out_features, m_pad, blocks):
    """Block-diagonal form of :func:`output_rht`."""
    _require_cuda(y_rht, "y_rht")
    bl = _blocks(blocks, m_pad)
    lib = _lib.load()
    if len(bl) > _lib.MAX_BLOCKS:
        raise RuntimeError(f"glq_b200: at most {_lib.MAX_BLOCKS} Hadamard blocks per transform")
    _lib.check(lib.glqb_output_rht(y_rht.data_ptr(), su.data_ptr(), out.data_ptr(), _dt(out.dtype), out.stride(0),
                                   int(out_features), int(m_pad), (C.c_int32 * len(bl))(*bl), len(bl),
                                   y_rht.shape[0], _stream(out)), "output_rht")


# ------------------------------------------------------------------------------------------------
# decode dumps and probes (glq/csrc/glq_bindings.cpp:345-352)
# ------------------------------------------------------------------------------------------------
def glq_trellis_kernel_supported(m: int, k: int) -> bool:
    return bool(_lib.load().glqb_trellis_kernel_supported(int(m), int(k)))


def glq_decompress_trellis_3inst_cuda(packed, m, k, allow_r1=True):
    """packed trellis -> dense fp16 (m, k), bit-exact with glq.trellis.decode_layer."""
    _require_cuda(packed, "packed")
    out = torch.empty(m, k, dtype=torch.float16, device=packed.device)
    _lib.check(_lib.load().glqb_decompress_trellis_3inst(packed.data_ptr(), _trellis_bits(packed), None, 0, 0.0,
                                                         int(m), int(k), out.data_ptr(), _lib.DT_F16,
                                                         _stream(packed)), "decompress_trellis_3inst")
    return out


def decompress_trellis_3inst_rvq2(packed, packed2, inv_resid_scale2, m, k):
    """fp32 (m, k) = dec(stage1) + dec(stage2) * inv_resid_scale2 (glq/trellis.py:923-933)."""
    out = torch.empty(m, k, dtype=torch.float32, device=packed.device)
    _lib.check(_lib.load().glqb_decompress_trellis_3inst(packed.data_ptr(), _trellis_bits(packed),
                                                         packed2.data_ptr(), _trellis_bits(packed2),
                                                         float(inv_resid_scale2), int(m), int(k), out.data_ptr(),
                                                         _lib.DT_F32, _stream(packed)), "decompress_trellis_3inst")
    return out


def dequant_e8(qidxs_list: Sequence[torch.Tensor], codebooks: Sequence[torch.Tensor],
               inv_resid_scales: Sequence[float]) -> torch.Tensor:
    """fp32 (m, n) rotated-domain weights the E8 kernels reconstruct (glq/quantized_linear.py:1177-1194)."""
    ns = len(qidxs_list)
    m, n = qidxs_list[0].shape[0], qidxs_list[0].shape[1] * 8
    tabs = [e8_packed_table(cb) for cb in codebooks]
    vp = C.c_void_p
    q = (vp * ns)(*[t.data_ptr() for t in qidxs_list])
    tb = (vp * ns)(*[t.data_ptr() for t in tabs])
    ent = (C.c_int32 * ns)(*[t.numel() for t in tabs])
    sc = (C.c_float * ns)(1.0, *[float(s) for s in inv_resid_scales])
    out = torch.empty(m, n, dtype=torch.float32, device=qidxs_list[0].device)
    _lib.check(_lib.load().glqb_dequant_e8(q, tb, ent, sc, ns, m, n, out.data_ptr(), _stream(out)), "dequant_e8")
    return out


# ------------------------------------------------------------------------------------------------
# MoE grouped expert matmul (glq_vllm/custom_ops.py:22-36)
# ------------------------------------------------------------------------------------------------
class MoePlan:
    """Owns a GlqbMoePlan handle and its workspace."""

    def __init__(self, desc: "_lib.MoeDesc", device, keep):
        self.lib = _lib.load()
        self.keep = keep
        handle = C.c_void_p()
        with torch.cuda.device(device):
            _lib.check(self.lib.glqb_moe_plan_create(C.byref(desc), C.byref(handle)), "moe_plan_create")
        self.handle = handle
        self.max_tokens = desc.max_tokens
        self.workspace = torch.empty(max(256, int(self.lib.glqb_moe_plan_workspace_bytes(handle))), dtype=torch.uint8,
                                     device=device)
        self.code_bytes = int(self.lib.glqb_moe_plan_code_bytes(handle))

    def run(self, x, topk_ids, topk_weights, y):
        _lib.check(self.lib.glqb_moe_plan_run(self.handle, x.data_ptr(), topk_ids.data_ptr(), topk_weights.data_ptr(),
                                              y.data_ptr(), x.shape[0], self.workspace.data_ptr(),
                                              self.workspace.numel(), _stream(x)), "moe_plan_run")

    def check_status(self, x=None):
        """Synchronises the stream of ``x`` (default: the current stream of the plan's device) and raises if a
        bounded wait inside the GEMM kernels gave up."""
        _lib.check(self.lib.glqb_moe_plan_status(self.handle, self.workspace.data_ptr(),
                                                 _stream(x if x is not None else self.workspace)), "moe_plan_status")

    def set_timing(self, on: bool) -> None:
        _lib.check(self.lib.glqb_moe_plan_set_timing(self.handle, 1 if on else 0), "moe_plan_set_timing")

    def kernel_ms(self):
        """(summed time of the two expert matmuls in ms, runs recorded) since timing was enabled; synchronises."""
        ms, runs = C.c_double(), C.c_int32()
        _lib.check(self.lib.glqb_moe_plan_kernel_ms(self.handle, C.byref(ms), C.byref(runs)), "moe_plan_kernel_ms")
        return float(ms.value), int(runs.value)

    def close(self):
        if getattr(self, "handle", None):
            self.lib.glqb_moe_plan_destroy(self.handle)
            self.handle = None


def _moe_capacity(tokens: int) -> int:
    cap = 16
    while cap < tokens:
        cap *= 2
    return cap


def fused_moe_trellis_3inst(x, topk_ids, topk_weights,
                            w13_trellis_packed, w13_trellis_packed2, w13_SU, w13_SV, w13_Wscale, w13_inv_resid_scale2,
                            w2_trellis_packed, w2_trellis_packed2, w2_SU, w2_SV, w2_Wscale, w2_inv_resid_scale2,
                            hidden_size, intermediate_size, w13_out_features,
                            n_pad_w13, m_pad_w13, n_pad_w2, m_pad_w2,
                            blocks_n_w13, blocks_m_w13, blocks_n_w13_meta, blocks_m_w13_meta,
                            blocks_n_w2, blocks_m_w2, blocks_n_w2_meta, blocks_m_w2_meta, activation_type,
                            out_dtype=None):
    """(T, hidden) -> (T, hidden): routed experts, gated activation, weighted combine; any token count,
    no host synchronisation.  A second-stage tensor with numel() <= E is the reference's "absent" sentinel.
    ``out_dtype`` (not in the reference) selects the result dtype, e.g. fp32 partial results of one
    expert-parallel rank; default: the dtype of x."""
    _require_cuda(x, "x")
    E = w13_trellis_packed.shape[0]
    T = x.shape[0]
    if T == 0:
        return torch.empty_like(x)
    x = x.contiguous()
    ids = topk_ids.contiguous()
    if ids.dtype not in (torch.int32, torch.int64):
        ids = ids.to(torch.int64)
    tw = topk_weights.to(torch.float32).contiguous()
    has13 = w13_trellis_packed2 is not None and w13_trellis_packed2.numel() > E
    has2 = w2_trellis_packed2 is not None and w2_trellis_packed2.numel() > E
    cap = _moe_capacity(T)
    odt = out_dtype or x.dtype
    key = ("moe3", w13_trellis_packed.data_ptr(), w2_trellis_packed.data_ptr(), cap, ids.shape[1], x.dtype, ids.dtype,
           int(activation_type), has13, has2, odt)
    plan = _PLAN_CACHE.get(key)
    if plan is not None:
        _PLAN_CACHE.move_to_end(key)
    if plan is None:
        d = _lib.MoeDesc()
        d.num_experts, d.top_k, d.hidden, d.inter, d.w13_out = E, ids.shape[1], hidden_size, intermediate_size, w13_out_features
        d.max_tokens, d.activation = cap, int(activation_type)
        d.w13_bits, d.w2_bits = w13_trellis_packed.shape[-1] // 16, w2_trellis_packed.shape[-1] // 16
        d.w13_bits2 = w13_trellis_packed2.shape[-1] // 16 if has13 else 0
        d.w2_bits2 = w2_trellis_packed2.shape[-1] // 16 if has2 else 0
        ws13 = w13_Wscale.to(torch.float32).contiguous()
        ws2 = w2_Wscale.to(torch.float32).contiguous()
        i13 = w13_inv_resid_scale2.to(torch.float32).contiguous() if has13 else None
        i2 = w2_inv_resid_scale2.to(torch.float32).contiguous() if has2 else None
        d.w13_packed, d.w13_packed2 = w13_trellis_packed.data_ptr(), (w13_trellis_packed2.data_ptr() if has13 else None)
        d.w13_su, d.w13_sv, d.w13_wscale = w13_SU.data_ptr(), w13_SV.data_ptr(), ws13.data_ptr()
        d.w13_inv_resid_scale2 = i13.data_ptr() if has13 else None
        d.w2_packed, d.w2_packed2 = w2_trellis_packed.data_ptr(), (w2_trellis_packed2.data_ptr() if has2 else None)
        d.w2_su, d.w2_sv, d.w2_wscale = w2_SU.data_ptr(), w2_SV.data_ptr(), ws2.data_ptr()
        d.w2_inv_resid_scale2 = i2.data_ptr() if has2 else None
        _fill_moe_blocks(d, blocks_n_w13, n_pad_w13, blocks_m_w13, m_pad_w13, blocks_n_w2, n_pad_w2, blocks_m_w2, m_pad_w2)
        d.ids_are_int64 = 1 if ids.dtype == torch.int64 else 0
        d.x_dtype, d.y_dtype = _dt(x.dtype), _dt(odt)
        plan = MoePlan(d, x.device, [w13_trellis_packed, w13_trellis_packed2, w13_SU, w13_SV, ws13, i13,
                                     w2_trellis_packed, w2_trellis_packed2, w2_SU, w2_SV, ws2, i2])
        _PLAN_CACHE[key] = plan
    y = torch.empty(T, hidden_size, dtype=odt, device=x.device)
    plan.run(x, ids, tw, y)
    return y


def _fill_moe_blocks(d, blocks_n_w13, n_pad_w13, blocks_m_w13, m_pad_w13, blocks_n_w2, n_pad_w2, blocks_m_w2, m_pad_w2):
    for name, blocks, total in (("n_w13", blocks_n_w13, n_pad_w13), ("m_w13", blocks_m_w13, m_pad_w13),
                                ("n_w2", blocks_n_w2, n_pad_w2), ("m_w2", blocks_m_w2, m_pad_w2)):
        bl = _blocks(blocks, total)
        setattr(d, "n_blocks_" + name, len(bl))
        arr = getattr(d, "blocks_" + name)
        for i, b in enumerate(bl):
            arr[i] = b


def fused_moe_grouped_gemm(x, topk_ids, topk_weights,
                           w13_Qidxs, w13_SU, w13_SV, w13_Wscale, w13_Qidxs2, w13_inv_rs,
                           w2_Qidxs, w2_SU, w2_SV, w2_Wscale, w2_Qidxs2, w2_inv_rs,
                           codebook, codebook2,
                           hidden_size, intermediate_size, w13_out_features,
                           n_pad_w13, m_pad_w13, n_pad_w2, m_pad_w2,
                           blocks_n_w13, blocks_m_w13, blocks_n_w13_meta, blocks_m_w13_meta,
                           blocks_n_w2, blocks_m_w2, blocks_n_w2_meta, blocks_m_w2_meta, activation_type,
                           w13_Qidxs3=None, w13_inv_rs2=None, w2_Qidxs3=None, w2_inv_rs2=None, codebook3=None):
    """E8-shell routed experts (glq_vllm/custom_ops.py:203-246): (T, hidden) -> (T, hidden).  Every expert is
    an E8 layer (m_pad, n_pad/8) of up to three stages with per-expert Wscale and inverse residual scales; a
    stage is present when its index tensor has the full (E, m_pad, n_pad/8) shape (the reference keeps an
    (E,1,1) placeholder otherwise).  Any token count; gated (0-2) and plain (3-5) activations."""
    _require_cuda(x, "x")
    E = w13_Qidxs.shape[0]
    T = x.shape[0]
    if T == 0:
        return torch.empty_like(x)
    if m_pad_w13 != w13_out_features or n_pad_w13 != hidden_size or n_pad_w2 != intermediate_size or m_pad_w2 != hidden_size:
        raise RuntimeError("glq_b200: E8 experts padded to powers of two are not served (block-diagonal layers only)")
    x = x.contiguous()
    ids = topk_ids.contiguous()
    if ids.dtype not in (torch.int32, torch.int64):
        ids = ids.to(torch.int64)
    tw = topk_weights.to(torch.float32).contiguous()
    full13, full2 = w13_Qidxs.numel(), w2_Qidxs.numel()
    stages13 = [(w13_Qidxs, None, codebook)]
    stages2 = [(w2_Qidxs, None, codebook)]
    for q13, i13, q2, i2, cb in ((w13_Qidxs2, w13_inv_rs, w2_Qidxs2, w2_inv_rs, codebook2),
                                 (w13_Qidxs3, w13_inv_rs2, w2_Qidxs3, w2_inv_rs2, codebook3)):
        ok = (q13 is not None and q2 is not None and cb is not None and i13 is not None and i2 is not None and
              q13.numel() == full13 and q2.numel() == full2 and cb.numel() > 0 and i13.numel() == E and i2.numel() == E)
        if not ok:
            break
        stages13.append((q13, i13.to(torch.float32).contiguous(), cb))
        stages2.append((q2, i2.to(torch.float32).contiguous(), cb))
    ns = len(stages13)
    cap = _moe_capacity(T)
    key = ("moe_e8", tuple(s[0].data_ptr() for s in stages13), tuple(s[0].data_ptr() for s in stages2), cap,
           ids.shape[1], x.dtype, ids.dtype, int(activation_type))
    plan = _PLAN_CACHE.get(key)
    if plan is None:
        d = _lib.MoeDesc()
        d.format, d.e8_stages = _lib.FMT_E8_SHELL, ns
        d.num_experts, d.top_k, d.hidden, d.inter, d.w13_out = E, ids.shape[1], hidden_size, intermediate_size, w13_out_features
        d.max_tokens, d.activation = cap, int(activation_type)
        ws13 = w13_Wscale.to(torch.float32).contiguous()
        ws2 = w2_Wscale.to(torch.float32).contiguous()
        tables = [e8_packed_table(s[2]) for s in stages13]
        for s in range(ns):
            d.w13_qidxs[s] = stages13[s][0].data_ptr()
            d.w2_qidxs[s] = stages2[s][0].data_ptr()
            d.e8_table[s] = tables[s].data_ptr()
            d.e8_table_entries[s] = tables[s].numel()
            if s:
                d.w13_inv_rs[s - 1] = stages13[s][1].data_ptr()
                d.w2_inv_rs[s - 1] = stages2[s][1].data_ptr()
        d.w13_su, d.w13_sv, d.w13_wscale = w13_SU.data_ptr(), w13_SV.data_ptr(), ws13.data_ptr()
        d.w2_su, d.w2_sv, d.w2_wscale = w2_SU.data_ptr(), w2_SV.data_ptr(), ws2.data_ptr()
        _fill_moe_blocks(d, blocks_n_w13, n_pad_w13, blocks_m_w13, m_pad_w13, blocks_n_w2, n_pad_w2, blocks_m_w2, m_pad_w2)
        d.ids_are_int64 = 1 if ids.dtype == torch.int64 else 0
        d.x_dtype = d.y_dtype = _dt(x.dtype)
        plan = MoePlan(d, x.device, [stages13, stages2, tables, w13_SU, w13_SV, ws13, w2_SU, w2_SV, ws2])
        _PLAN_CACHE[key] = plan
    else:
        _PLAN_CACHE.move_to_end(key)
    y = torch.empty(T, hidden_size, dtype=x.dtype, device=x.device)
    plan.run(x, ids, tw, y)
    return y


# the reference's per-(token, expert) op has the same signature and result (glq_vllm/custom_ops.py:203-224)
fused_moe_block_diag = fused_moe_grouped_gemm

glq_fused_moe_trellis_3inst_cuda = fused_moe_trellis_3inst
glq_fused_moe_grouped_gemm_cuda = fused_moe_grouped_gemm
glq_fused_moe_block_diag_cuda = fused_moe_block_diag

# names under which the reference's extension module exposes the same entry points
glq_fused_linear_cuda = fused_linear
glq_fused_linear_block_diag_cuda = fused_linear_block_diag
glq_fused_linear_trellis_3inst_cuda = fused_linear_trellis_3inst
glq_fused_linear_trellis_3inst_rvq2_cuda = fused_linear_trellis_3inst_rvq2
glq_fused_linear_trellis_3inst_yrht_cuda = fused_linear_trellis_3inst_yrht
glq_fused_linear_trellis_3inst_yrht_rvq2_cuda = fused_linear_trellis_3inst_yrht_rvq2
glq_output_rht_shards_cuda = output_rht_shards
glq_dequant_matvec_cuda = dequant_matvec
glq_dequant_matmul_cuda = dequant_matmul
glq_input_rht_cuda = input_rht
glq_output_rht_cuda = output_rht
