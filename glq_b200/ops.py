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
import math
from typing import Optional, Sequence

import torch

from . import _lib
from .plan import LinearSpec, Plan, block_decompose

DECODE_MAX_TOKENS = 64
_PLAN_CACHE: dict = {}
_TABLE_CACHE: dict = {}


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
    key = (codebook.data_ptr(), codebook.shape[0], codebook.device.index)
    tb = _TABLE_CACHE.get(key)
    if tb is None:
        cb = codebook.to(torch.float16).contiguous()
        tb = torch.empty(cb.shape[0], dtype=torch.int32, device=cb.device)
        _lib.check(_lib.load().glqb_e8_pack_table(cb.data_ptr(), cb.shape[0], tb.data_ptr(), _stream(cb)),
                   "e8_pack_table")
        _TABLE_CACHE[key] = tb
    return tb


def _cached_plan(key, make_specs) -> Plan:
    p = _PLAN_CACHE.get(key)
    if p is None:
        p = Plan(make_specs())
        _PLAN_CACHE[key] = p
    return p


def clear_caches() -> None:
    for p in _PLAN_CACHE.values():
        p.close()
    _PLAN_CACHE.clear()
    _TABLE_CACHE.clear()


def _run_sliced(x2d: torch.Tensor, out: torch.Tensor, key_base, make_spec, max_tokens=DECODE_MAX_TOKENS) -> None:
    """Run a single-layer op over x2d (B, in) -> out (B, out) in slices of <= max_tokens tokens."""
    B = x2d.shape[0]
    if B > DECODE_MAX_TOKENS:
        # prefill: one tensor-core GEMM plan for the whole token count
        plan = _cached_plan(key_base + (B, x2d.dtype, out.dtype, x2d.stride(0), out.stride(0)),
                            lambda: [make_spec(B)])
        plan.run(x2d, out)
        return
    done = 0
    while done < B:
        b = min(max_tokens, B - done)
        plan = _cached_plan(key_base + (b, x2d.dtype, out.dtype, x2d.stride(0), out.stride(0)),
                            lambda: [make_spec(b)])
        plan.run(x2d[done:], out[done:])
        done += b


# ------------------------------------------------------------------------------------------------
# trellis 3INST fused linears (glq_vllm/custom_ops.py:373-418)
# ------------------------------------------------------------------------------------------------
def _trellis_bits(packed: torch.Tensor) -> int:
    return packed.shape[-1] // 16


def _fused_trellis(x, sv, su, packed, packed2, blocks_n, blocks_m, wscale, inv_rs2, in_features,
                   out_features, n_pad, m_pad, y_rht_out=None, col=0, out_dtype=None):
    _require_cuda(x, "x")
    x2d = x.reshape(-1, in_features)
    if x2d.stride(-1) != 1:
        x2d = x2d.contiguous()
    has2 = packed2 is not None and packed2.numel() > 0
    codes = [packed] + ([packed2] if has2 else [])
    bits = [_trellis_bits(packed)] + ([_trellis_bits(packed2)] if has2 else [])
    bn, bm = _blocks(blocks_n, n_pad), _blocks(blocks_m, m_pad)
    if y_rht_out is None:
        out = torch.empty(x2d.shape[0], out_features, dtype=out_dtype or x2d.dtype, device=x2d.device)
        tgt, yoff, stop = out, 0, False
    else:
        tgt, yoff, stop = y_rht_out, int(col), True

    def make_spec(b):
        return LinearSpec(format=_lib.FMT_TRELLIS_3INST, m_pad=m_pad, n_pad=n_pad, in_features=in_features,
                          out_features=out_features if not stop else m_pad, codes=codes, bits=bits, su=su, sv=sv,
                          wscale=float(wscale), stage_scale=[float(inv_rs2)] if has2 else [],
                          blocks_n=bn, blocks_m=bm, batch=b, x_dtype=x2d.dtype, y_dtype=tgt.dtype,
                          x_stride=x2d.stride(0), y_stride=tgt.stride(0), y_offset=yoff, stop_at_yrht=stop)

    key = ("trellis", packed.data_ptr(), packed2.data_ptr() if has2 else 0, su.data_ptr() if su is not None else 0,
           sv.data_ptr(), float(wscale), float(inv_rs2), m_pad, n_pad, out_features, stop, yoff)
    # two decoded stages keep two accumulator sets: 32 tokens per pass instead of 64
    _run_sliced(x2d, tgt, key, make_spec, 32 if has2 else DECODE_MAX_TOKENS)
    return None if stop else tgt


def fused_linear_trellis_3inst(x, sv, su, trellis_packed, blocks_n, blocks_m, blocks_n_meta, blocks_m_meta,
                               wscale, in_features, out_features, n_pad, m_pad, out_dtype=None):
    """input RHT -> 3INST decode + matmul -> x Wscale -> output RHT, (B, in) -> (B, out).
    ``out_dtype`` (not in the reference) selects the result dtype; default: the dtype of x."""
    return _fused_trellis(x, sv, su, trellis_packed, None, blocks_n, blocks_m, wscale, 0.0,
                          in_features, out_features, n_pad, m_pad, out_dtype=out_dtype)


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
    shard_meta rows are (global column offset, block size, log2, optional normalisation bits)."""
    _require_cuda(y_rht, "y_rht")
    meta = shard_meta.cpu().tolist() if isinstance(shard_meta, torch.Tensor) else list(shard_meta)
    blocks = [int(r[1]) for r in meta]
    total = sum(blocks)
    B = y_rht.shape[0]
    arr = (C.c_int32 * len(blocks))(*blocks)
    _lib.check(_lib.load().glqb_output_rht(y_rht.data_ptr(), su.data_ptr(), y.data_ptr(), _dt(y.dtype), y.stride(0),
                                           int(out_features), total, arr, len(blocks), B, _stream(y)),
               "output_rht_shards")


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
              x_is_rotated=False, stop=False, out_dtype=None):
    _require_cuda(x, "x")
    feat_in = n_pad if x_is_rotated else in_features
    x2d = x.reshape(-1, feat_in)
    if x2d.stride(-1) != 1:
        x2d = x2d.contiguous()
    odt = torch.float32 if stop else (out_dtype or x2d.dtype)
    out = torch.empty(x2d.shape[0], m_pad if stop else out_features, dtype=odt, device=x2d.device)

    def make_spec(b):
        return LinearSpec(format=_lib.FMT_E8_SHELL, m_pad=m_pad, n_pad=n_pad, in_features=feat_in,
                          out_features=m_pad if stop else out_features, codes=codes, tables=tables,
                          stage_scale=scales, su=su, sv=sv, wscale=float(wscale), blocks_n=bn, blocks_m=bm,
                          batch=b, x_dtype=x2d.dtype, y_dtype=odt, x_stride=x2d.stride(0), y_stride=out.stride(0),
                          stop_at_yrht=stop, x_is_rotated=x_is_rotated)

    key = ("e8", tuple(c.data_ptr() for c in codes), tuple(t.data_ptr() for t in tables), tuple(scales),
           su.data_ptr(), sv.data_ptr(), float(wscale), m_pad, n_pad, in_features, out_features, stop, x_is_rotated)
    _run_sliced(x2d, out, key, make_spec, 32 if len(codes) > 2 else DECODE_MAX_TOKENS)
    return out


_EMPTY = None


def fused_linear(x, sv, su, qidxs, codebook, wscale, in_features, out_features, n_pad, m_pad, log_n, log_m,
                 qidxs2=_EMPTY, codebook2=_EMPTY, inv_resid_scale=0.0, qidxs3=_EMPTY, codebook3=_EMPTY,
                 inv_resid_scale2=0.0, qidxs4=_EMPTY, codebook4=_EMPTY, inv_resid_scale3=0.0, out_dtype=None):
    """Power-of-two padded E8 layer: whole-length Hadamard on both sides."""
    codes, tables, scales = _e8_stages(qidxs, codebook, qidxs2, codebook2, inv_resid_scale, qidxs3, codebook3,
                                       inv_resid_scale2, qidxs4, codebook4, inv_resid_scale3)
    return _fused_e8(x, sv, su, codes, tables, scales, wscale, in_features, out_features, n_pad, m_pad,
                     [n_pad], [m_pad], out_dtype=out_dtype)


def fused_linear_block_diag(x, sv, su, qidxs, codebook, wscale, in_features, out_features, n_pad, m_pad,
                            blocks_n, blocks_m, blocks_n_meta, blocks_m_meta,
                            qidxs2=_EMPTY, codebook2=_EMPTY, inv_resid_scale=0.0, qidxs3=_EMPTY, codebook3=_EMPTY,
                            inv_resid_scale2=0.0, qidxs4=_EMPTY, codebook4=_EMPTY, inv_resid_scale3=0.0,
                            out_dtype=None):
    """Unpadded E8 layer with block-diagonal Hadamards."""
    codes, tables, scales = _e8_stages(qidxs, codebook, qidxs2, codebook2, inv_resid_scale, qidxs3, codebook3,
                                       inv_resid_scale2, qidxs4, codebook4, inv_resid_scale3)
    return _fused_e8(x, sv, su, codes, tables, scales, wscale, in_features, out_features, n_pad, m_pad,
                     _blocks(blocks_n, n_pad), _blocks(blocks_m, m_pad), out_dtype=out_dtype)


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

    def check_status(self, x):
        """Synchronises the stream of ``x`` and raises if a bounded wait inside the GEMM kernels gave up."""
        _lib.check(self.lib.glqb_moe_plan_status(self.handle, self.workspace.data_ptr(), _stream(x)), "moe_plan_status")

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
                            blocks_n_w2, blocks_m_w2, blocks_n_w2_meta, blocks_m_w2_meta, activation_type):
    """(T, hidden) -> (T, hidden): routed experts, gated activation, weighted combine; any token count,
    no host synchronisation.  A second-stage tensor with numel() <= E is the reference's "absent" sentinel."""
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
    key = ("moe3", w13_trellis_packed.data_ptr(), w2_trellis_packed.data_ptr(), cap, ids.shape[1], x.dtype, ids.dtype,
           int(activation_type), has13, has2)
    plan = _PLAN_CACHE.get(key)
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
        for name, blocks, total in (("n_w13", blocks_n_w13, n_pad_w13), ("m_w13", blocks_m_w13, m_pad_w13),
                                    ("n_w2", blocks_n_w2, n_pad_w2), ("m_w2", blocks_m_w2, m_pad_w2)):
            bl = _blocks(blocks, total)
            setattr(d, "n_blocks_" + name, len(bl))
            arr = getattr(d, "blocks_" + name)
            for i, b in enumerate(bl):
                arr[i] = b
        d.ids_are_int64 = 1 if ids.dtype == torch.int64 else 0
        d.x_dtype = d.y_dtype = _dt(x.dtype)
        plan = MoePlan(d, x.device, [w13_trellis_packed, w13_trellis_packed2, w13_SU, w13_SV, ws13, i13,
                                     w2_trellis_packed, w2_trellis_packed2, w2_SU, w2_SV, ws2, i2])
        _PLAN_CACHE[key] = plan
    y = torch.empty(T, hidden_size, dtype=x.dtype, device=x.device)
    plan.run(x, ids, tw, y)
    return y


glq_fused_moe_trellis_3inst_cuda = fused_moe_trellis_3inst

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
