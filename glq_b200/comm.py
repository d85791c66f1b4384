"""Sums over tensor-parallel ranks inside the library's own kernels (``glqb_comm_*`` of the C ABI).

The reference leaves the sum of row-parallel partial outputs (o_proj, down_proj) to its host framework's NCCL
all-reduce (glq_vllm/linear_method.py:1031-1102 under vLLM's RowParallelLinear).  For decode-sized outputs that
call is all latency; a :class:`Comm` lets the decode kernel (or one small stand-alone launch) do the sum through
NVLink stores into every rank's receive area instead.  One process per GPU, all ranks on one node.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib

HANDLE_BYTES = 64


class Comm:
    """One rank's end of a communicator.  ``Comm.from_process_group`` builds and connects it across the ranks of a
    ``torch.distributed`` group; ``Comm.local_group`` builds all ranks inside one process (tests, or one process
    that drives several GPUs)."""

    def __init__(self, rank: int, world: int, max_floats: int = 1 << 16, device: Optional[torch.device] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("glq_b200.comm needs a CUDA device")
        self.lib = _lib.load()
        self.rank, self.world, self.max_floats = int(rank), int(world), int(max_floats)
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.handle = C.c_void_p()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.glqb_comm_create(self.rank, self.world, self.max_floats, C.byref(self.handle)), "comm_create")

    # ---- set-up ---------------------------------------------------------------------------------------
    def ipc_handle(self) -> bytes:
        buf = C.create_string_buffer(HANDLE_BYTES)
        _lib.check(self.lib.glqb_comm_handle(self.handle, buf, HANDLE_BYTES), "comm_handle")
        return buf.raw

    def connect(self, handles: Sequence[bytes]) -> None:
        if len(handles) != self.world or any(len(h) != HANDLE_BYTES for h in handles):
            raise ValueError(f"need {self.world} handles of {HANDLE_BYTES} bytes")
        blob = b"".join(handles)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.glqb_comm_connect(self.handle, blob, HANDLE_BYTES), "comm_connect")

    @classmethod
    def from_process_group(cls, group=None, max_floats: int = 1 << 16, device=None) -> "Comm":
        import torch.distributed as dist
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        c = cls(rank, world, max_floats, device)
        if world > 1:
            handles: list = [None] * world
            dist.all_gather_object(handles, c.ipc_handle(), group=group)
            c.connect(handles)
            dist.barrier(group=group)
        return c

    @classmethod
    def local_group(cls, world: int, max_floats: int = 1 << 16, devices: Optional[Sequence] = None) -> list["Comm"]:
        devices = list(devices) if devices is not None else [torch.device("cuda", torch.cuda.current_device())] * world
        comms = [cls(r, world, max_floats, devices[r]) for r in range(world)]
        arr = (C.c_void_p * world)(*[c.handle for c in comms])
        for c in comms:
            with torch.cuda.device(c.device):
                _lib.check(c.lib.glqb_comm_connect_local(c.handle, arr), "comm_connect_local")
        return comms

    def set_timeout_ms(self, ms: int) -> None:
        _lib.check(self.lib.glqb_comm_set_timeout_ms(self.handle, int(ms)), "comm_set_timeout_ms")

    # ---- use ------------------------------------------------------------------------------------------
    def all_reduce_(self, buf: torch.Tensor) -> torch.Tensor:
        """In-place sum of a dense fp32 tensor of at most ``max_floats`` values over the ranks (one launch on the
        current stream; every rank must call it in the same order relative to the other uses of this object)."""
        if buf.dtype != torch.float32 or not buf.is_contiguous() or not buf.is_cuda:
            raise RuntimeError("glq_b200.comm: all_reduce_ takes a dense fp32 CUDA tensor")
        stream = torch.cuda.current_stream(buf.device).cuda_stream
        _lib.check(self.lib.glqb_comm_all_reduce(self.handle, buf.data_ptr(), buf.numel(), stream), "comm_all_reduce")
        return buf

    def status(self, reset: bool = False) -> int:
        """Synchronising read of the status word: 0, or 6 after a wait for a peer ran out (the results of that launch
        are invalid; the context stays usable)."""
        v = C.c_int32(0)
        self.lib.glqb_comm_status(self.handle, C.byref(v), 1 if reset else 0)
        return int(v.value)

    def check_status(self) -> None:
        v = C.c_int32(0)
        _lib.check(self.lib.glqb_comm_status(self.handle, C.byref(v), 0), "comm_status")

    def epoch(self) -> int:
        v = C.c_int32(0)
        _lib.check(self.lib.glqb_comm_epoch(self.handle, C.byref(v)), "comm_epoch")
        return int(v.value)

    def close(self) -> None:
        if self.handle:
            self.lib.glqb_comm_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass
