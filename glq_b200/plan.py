"""Host-side description of quantised linears and the plan object that runs them.

A *plan* is a fixed set of independent GLQ linears (for example the q/k/v shards of one attention
block, the gate/up shards of an MLP, the experts of a MoE step, or every projection of a model in
a sweep) executed by one short, allocation-free launch sequence.  Plans are built once — the
analogue of the reference's ``process_weights_after_loading`` (glq_vllm/linear_method.py:1031),
which hoists every host-side decision out of ``apply`` — and then run many times, also under
CUDA-graph capture.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from . import _lib

_DT = {torch.float16: _lib.DT_F16, torch.bfloat16: _lib.DT_BF16, torch.float32: _lib.DT_F32}


def block_decompose(n: int) -> list[int]:
    """Descending powers of two summing to n (glq/hadamard.py:133-146)."""
    out = []
    while n > 0:
        p = 1 << (n.bit_length() - 1)
        out.append(p)
        n -= p
    return out


@dataclass
class LinearSpec:
    """One GLQ linear in the reference's storage (glq/quantized_linear.py:235-247, 351-361)."""
    format: int                                   # _lib.FMT_TRELLIS_3INST or _lib.FMT_E8_SHELL
    m_pad: int
    n_pad: int
    in_features: int
    out_features: int
    codes: Sequence[torch.Tensor]                 # per stage: trellis_packed{,2} or Qidxs{,2,3,4}
    su: torch.Tensor
    sv: torch.Tensor
    wscale: float
    bits: Sequence[int] = ()                      # trellis: K per stage
    tables: Sequence[Optional[torch.Tensor]] = () # E8: packed uint32 (as int32 tensor) table per stage
    stage_scale: Sequence[float] = ()             # cumulative inverse residual scales, stages 2..
    blocks_n: Optional[Sequence[int]] = None
    blocks_m: Optional[Sequence[int]] = None
    row_scale: Optional[torch.Tensor] = None
    batch: int = 1
    x_dtype: torch.dtype = torch.bfloat16
    y_dtype: torch.dtype = torch.bfloat16
    x_stride: Optional[int] = None
    y_stride: Optional[int] = None
    x_offset: int = 0
    y_offset: int = 0
    stop_at_yrht: bool = False
    x_is_rotated: bool = False
    # fusions of the single-launch decode form (at most 8 tokens; plan creation refuses them otherwise)
    in_norm_weight: Optional[torch.Tensor] = None  # RMSNorm weight (in_features,), fp16 / bf16 / fp32
    in_norm_eps: float = 1e-6
    in_gated_act: Optional[int] = None             # 0 silu, 1 gelu-tanh, 2 relu^2: x rows hold [gate | up]
    y_accumulate: bool = False                     # y <- y + result (residual add)
    keep: list = field(default_factory=list)      # tensors kept alive for the plan

    def to_desc(self) -> _lib.LinearDesc:
        d = _lib.LinearDesc()
        d.format = self.format
        d.m_pad, d.n_pad = self.m_pad, self.n_pad
        d.in_features, d.out_features = self.in_features, self.out_features
        d.n_stages = len(self.codes)
        for s, t in enumerate(self.codes):
            if not t.is_cuda or not t.is_contiguous():
                raise RuntimeError("glq_b200: code tensors must be contiguous CUDA tensors")
            d.codes[s] = t.data_ptr()
            if self.format == _lib.FMT_TRELLIS_3INST:
                d.bits[s] = int(self.bits[s])
            else:
                tb = self.tables[s]
                d.table[s] = tb.data_ptr()
                d.table_entries[s] = tb.numel()
            if s:
                d.stage_scale[s] = float(self.stage_scale[s - 1])
        d.stage_scale[0] = 1.0
        d.wscale = float(self.wscale)
        d.row_scale = self.row_scale.data_ptr() if self.row_scale is not None else None
        for t in (self.su, self.sv):
            if t.dtype != torch.float16 or not t.is_cuda:
                raise RuntimeError("glq_b200: SU/SV must be fp16 CUDA tensors")
        d.su, d.sv = self.su.data_ptr(), self.sv.data_ptr()
        bn = list(self.blocks_n) if self.blocks_n is not None else block_decompose(self.n_pad)
        bm = list(self.blocks_m) if self.blocks_m is not None else block_decompose(self.m_pad)
        d.n_blocks_n, d.n_blocks_m = len(bn), len(bm)
        for i, b in enumerate(bn):
            d.blocks_n[i] = int(b)
        for i, b in enumerate(bm):
            d.blocks_m[i] = int(b)
        d.batch = self.batch
        d.x_dtype, d.y_dtype = _DT[self.x_dtype], _DT[self.y_dtype]
        d.x_stride = self.x_stride if self.x_stride is not None else self.in_features
        d.y_stride = self.y_stride if self.y_stride is not None else self.out_features
        d.x_offset, d.y_offset = self.x_offset, self.y_offset
        d.stop_at_yrht = 1 if self.stop_at_yrht else 0
        d.x_is_rotated = 1 if self.x_is_rotated else 0
        if self.in_norm_weight is not None:
            w = self.in_norm_weight
            if not w.is_cuda or not w.is_contiguous() or w.numel() != self.in_features:
                raise RuntimeError("glq_b200: the norm weight must be a contiguous CUDA tensor of in_features values")
            d.in_norm_weight, d.in_norm_dtype, d.in_norm_eps = w.data_ptr(), _DT[w.dtype], float(self.in_norm_eps)
        d.in_gated_act = 0 if self.in_gated_act is None else 1 + int(self.in_gated_act)
        d.y_accumulate = 1 if self.y_accumulate else 0
        return d


class Plan:
    """Owns a GlqbPlan handle and its workspace tensor."""

    def __init__(self, specs: Sequence[LinearSpec], device: Optional[torch.device] = None,
                 own_workspace: bool = True):
        self.lib = _lib.load()
        self.specs = list(specs)
        if not self.specs:
            raise RuntimeError("glq_b200: empty plan")
        self.device = device or self.specs[0].su.device
        arr = (_lib.LinearDesc * len(self.specs))(*[s.to_desc() for s in self.specs])
        handle = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.glqb_plan_create(arr, len(self.specs), C.byref(handle)), "plan_create")
        self.handle = handle
        self.workspace_bytes = int(self.lib.glqb_plan_workspace_bytes(handle))
        # own_workspace=False: the caller passes a (shared) workspace to every run
        self.workspace = (torch.empty(max(256, self.workspace_bytes), dtype=torch.uint8, device=self.device)
                          if own_workspace else None)
        self.code_bytes = int(self.lib.glqb_plan_code_bytes(handle))
        self.flops = int(self.lib.glqb_plan_flops(handle))
        self.launches = int(self.lib.glqb_plan_launches(handle))

    def run(self, x: torch.Tensor, y: torch.Tensor, stream: Optional[torch.cuda.Stream] = None,
            workspace: Optional[torch.Tensor] = None) -> None:
        """Enqueue on ``stream`` (default: the current torch stream); does not synchronise."""
        st = stream if stream is not None else torch.cuda.current_stream(self.device)
        ws = workspace if workspace is not None else self.workspace
        if ws is None:
            raise RuntimeError("glq_b200: this plan owns no workspace; pass one to run()")
        _lib.check(self.lib.glqb_plan_run(self.handle, x.data_ptr(), y.data_ptr(), ws.data_ptr(), ws.numel(),
                                          st.cuda_stream), "plan_run")

    def set_timing(self, on: bool) -> None:
        _lib.check(self.lib.glqb_plan_set_timing(self.handle, 1 if on else 0), "plan_set_timing")

    def kernel_ms(self) -> tuple[float, int]:
        """(summed decode-kernel time in ms, runs recorded) since timing was enabled; synchronises."""
        ms, runs = C.c_double(), C.c_int32()
        _lib.check(self.lib.glqb_plan_kernel_ms(self.handle, C.byref(ms), C.byref(runs)), "plan_kernel_ms")
        return float(ms.value), int(runs.value)

    def check_status(self) -> None:
        """Raise if a kernel of an earlier run gave up on a bounded wait (synchronises)."""
        st = C.c_int32()
        _lib.check(self.lib.glqb_plan_status(self.handle, C.byref(st)), "plan_status")

    def set_comm(self, comm) -> None:
        """The outputs of all layers become sums over the ranks of ``comm`` (a ``glq_b200.comm.Comm``), computed
        inside the single-launch decode kernel; raises RuntimeError for plans that do not take that form."""
        self._comm = comm                       # keeps the communicator alive as long as the plan points at it
        _lib.check(self.lib.glqb_plan_set_comm(self.handle, comm.handle if comm is not None else None), "plan_set_comm")

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.glqb_plan_destroy(self.handle)
            self.handle = None

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass
