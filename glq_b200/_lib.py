"""ctypes binding of libglq_b200.so (the C ABI declared in include/glq_b200.h).

There is no fallback: if the shared library is missing or a call fails, a RuntimeError is
raised (the reference raises through TORCH_CHECK, glq/csrc/glq_cuda.cu:27-29).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("GLQB_LIB_PATH") or os.path.join(_HERE, "libglq_b200.so")

MAX_STAGES = 4
MAX_BLOCKS = 16
FMT_TRELLIS_3INST = 0
FMT_E8_SHELL = 1
DT_F16, DT_BF16, DT_F32 = 0, 1, 2

EXPORTS = [
    "glqb_plan_create", "glqb_plan_workspace_bytes", "glqb_plan_code_bytes", "glqb_plan_flops",
    "glqb_plan_launches", "glqb_plan_run", "glqb_plan_set_timing", "glqb_plan_kernel_ms",
    "glqb_plan_destroy", "glqb_plan_status", "glqb_linear_workspace_bytes", "glqb_fused_linear",
    "glqb_decompress_trellis_3inst", "glqb_dequant_e8", "glqb_e8_pack_table", "glqb_input_rht",
    "glqb_output_rht", "glqb_output_rht_shards", "glqb_trellis_kernel_supported", "glqb_last_error", "glqb_version",
    "glqb_trellis_linear_noalloc", "glqb_noalloc_scratch_bytes",
    "glqb_moe_plan_create", "glqb_moe_plan_workspace_bytes", "glqb_moe_plan_code_bytes", "glqb_moe_plan_run",
    "glqb_moe_plan_status", "glqb_moe_plan_destroy", "glqb_moe_plan_set_timing", "glqb_moe_plan_kernel_ms",
    "glqb_comm_create", "glqb_comm_handle", "glqb_comm_connect", "glqb_comm_connect_local", "glqb_comm_set_timeout_ms",
    "glqb_comm_max_floats", "glqb_comm_all_reduce", "glqb_comm_status", "glqb_comm_epoch", "glqb_comm_destroy",
    "glqb_plan_set_comm",
]


class MoeDesc(C.Structure):
    _fields_ = [
        ("num_experts", C.c_int32), ("top_k", C.c_int32), ("hidden", C.c_int32), ("inter", C.c_int32),
        ("w13_out", C.c_int32), ("max_tokens", C.c_int32), ("activation", C.c_int32),
        ("w13_bits", C.c_int32), ("w13_bits2", C.c_int32), ("w2_bits", C.c_int32), ("w2_bits2", C.c_int32),
        ("w13_packed", C.c_void_p), ("w13_packed2", C.c_void_p), ("w13_su", C.c_void_p), ("w13_sv", C.c_void_p),
        ("w13_wscale", C.c_void_p), ("w13_inv_resid_scale2", C.c_void_p),
        ("w2_packed", C.c_void_p), ("w2_packed2", C.c_void_p), ("w2_su", C.c_void_p), ("w2_sv", C.c_void_p),
        ("w2_wscale", C.c_void_p), ("w2_inv_resid_scale2", C.c_void_p),
        ("n_blocks_n_w13", C.c_int32), ("n_blocks_m_w13", C.c_int32),
        ("n_blocks_n_w2", C.c_int32), ("n_blocks_m_w2", C.c_int32),
        ("blocks_n_w13", C.c_int32 * MAX_BLOCKS), ("blocks_m_w13", C.c_int32 * MAX_BLOCKS),
        ("blocks_n_w2", C.c_int32 * MAX_BLOCKS), ("blocks_m_w2", C.c_int32 * MAX_BLOCKS),
        ("ids_are_int64", C.c_int32), ("x_dtype", C.c_int32), ("y_dtype", C.c_int32),
        ("format", C.c_int32), ("e8_stages", C.c_int32),
        ("w13_qidxs", C.c_void_p * 3), ("w2_qidxs", C.c_void_p * 3), ("e8_table", C.c_void_p * 3),
        ("e8_table_entries", C.c_int32 * 3), ("w13_inv_rs", C.c_void_p * 2), ("w2_inv_rs", C.c_void_p * 2),
    ]


class LinearDesc(C.Structure):
    _fields_ = [
        ("format", C.c_int32),
        ("m_pad", C.c_int32), ("n_pad", C.c_int32),
        ("in_features", C.c_int32), ("out_features", C.c_int32),
        ("n_stages", C.c_int32),
        ("bits", C.c_int32 * MAX_STAGES),
        ("codes", C.c_void_p * MAX_STAGES),
        ("table", C.c_void_p * MAX_STAGES),
        ("table_entries", C.c_int32 * MAX_STAGES),
        ("stage_scale", C.c_float * MAX_STAGES),
        ("wscale", C.c_float),
        ("row_scale", C.c_void_p),
        ("su", C.c_void_p), ("sv", C.c_void_p),
        ("n_blocks_n", C.c_int32), ("n_blocks_m", C.c_int32),
        ("blocks_n", C.c_int32 * MAX_BLOCKS),
        ("blocks_m", C.c_int32 * MAX_BLOCKS),
        ("batch", C.c_int32),
        ("x_dtype", C.c_int32), ("y_dtype", C.c_int32),
        ("x_stride", C.c_int64), ("y_stride", C.c_int64),
        ("x_offset", C.c_int64), ("y_offset", C.c_int64),
        ("stop_at_yrht", C.c_int32), ("x_is_rotated", C.c_int32),
        ("in_norm_weight", C.c_void_p), ("in_norm_dtype", C.c_int32), ("in_norm_eps", C.c_float),
        ("in_gated_act", C.c_int32), ("y_accumulate", C.c_int32),
    ]


_lib = None


def load() -> C.CDLL:
    """Load the shared library (once). Raises RuntimeError when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m glq_b200.build` "
            "(nvcc, sm_100a). glq_b200 has no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    vp, i32, i64, f32, sz = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_size_t
    lib.glqb_plan_create.argtypes = [C.POINTER(LinearDesc), i32, C.POINTER(vp)]
    lib.glqb_plan_create.restype = C.c_int
    lib.glqb_plan_workspace_bytes.argtypes = [vp]
    lib.glqb_plan_workspace_bytes.restype = sz
    lib.glqb_plan_code_bytes.argtypes = [vp]
    lib.glqb_plan_code_bytes.restype = i64
    lib.glqb_plan_flops.argtypes = [vp]
    lib.glqb_plan_flops.restype = i64
    lib.glqb_plan_launches.argtypes = [vp]
    lib.glqb_plan_launches.restype = i32
    lib.glqb_plan_run.argtypes = [vp, vp, vp, vp, sz, vp]
    lib.glqb_plan_run.restype = C.c_int
    lib.glqb_plan_set_timing.argtypes = [vp, i32]
    lib.glqb_plan_set_timing.restype = C.c_int
    lib.glqb_plan_kernel_ms.argtypes = [vp, C.POINTER(C.c_double), C.POINTER(i32)]
    lib.glqb_plan_kernel_ms.restype = C.c_int
    lib.glqb_plan_status.argtypes = [vp, C.POINTER(i32)]
    lib.glqb_plan_status.restype = C.c_int
    lib.glqb_plan_destroy.argtypes = [vp]
    lib.glqb_plan_destroy.restype = None
    lib.glqb_linear_workspace_bytes.argtypes = [C.POINTER(LinearDesc)]
    lib.glqb_linear_workspace_bytes.restype = sz
    lib.glqb_fused_linear.argtypes = [C.POINTER(LinearDesc), vp, vp, vp, sz, vp]
    lib.glqb_fused_linear.restype = C.c_int
    lib.glqb_decompress_trellis_3inst.argtypes = [vp, i32, vp, i32, f32, i32, i32, vp, i32, vp]
    lib.glqb_decompress_trellis_3inst.restype = C.c_int
    lib.glqb_dequant_e8.argtypes = [C.POINTER(vp), C.POINTER(vp), C.POINTER(i32), C.POINTER(f32),
                                    i32, i32, i32, vp, vp]
    lib.glqb_dequant_e8.restype = C.c_int
    lib.glqb_e8_pack_table.argtypes = [vp, i32, vp, vp]
    lib.glqb_e8_pack_table.restype = C.c_int
    lib.glqb_input_rht.argtypes = [vp, i32, i64, vp, vp, i32, i32, C.POINTER(i32), i32, i32, vp]
    lib.glqb_input_rht.restype = C.c_int
    lib.glqb_output_rht.argtypes = [vp, vp, vp, i32, i64, i32, i32, C.POINTER(i32), i32, i32, vp]
    lib.glqb_output_rht.restype = C.c_int
    lib.glqb_output_rht_shards.argtypes = [vp, vp, vp, i32, i64, i32, i32, C.POINTER(i32), C.POINTER(i32), i32, i32, vp]
    lib.glqb_output_rht_shards.restype = C.c_int
    lib.glqb_trellis_kernel_supported.argtypes = [i32, i32]
    lib.glqb_trellis_kernel_supported.restype = C.c_int
    lib.glqb_trellis_linear_noalloc.argtypes = [vp, i32, vp, i32, vp, i32, vp, vp, f32, i32, i32,
                                                C.POINTER(i32), i32, C.POINTER(i32), i32, vp]
    lib.glqb_trellis_linear_noalloc.restype = C.c_int
    lib.glqb_noalloc_scratch_bytes.argtypes = []
    lib.glqb_noalloc_scratch_bytes.restype = sz
    lib.glqb_moe_plan_create.argtypes = [C.POINTER(MoeDesc), C.POINTER(vp)]
    lib.glqb_moe_plan_create.restype = C.c_int
    lib.glqb_moe_plan_workspace_bytes.argtypes = [vp]
    lib.glqb_moe_plan_workspace_bytes.restype = sz
    lib.glqb_moe_plan_code_bytes.argtypes = [vp]
    lib.glqb_moe_plan_code_bytes.restype = i64
    lib.glqb_moe_plan_run.argtypes = [vp, vp, vp, vp, vp, i32, vp, sz, vp]
    lib.glqb_moe_plan_run.restype = C.c_int
    lib.glqb_moe_plan_status.argtypes = [vp, vp, vp]
    lib.glqb_moe_plan_status.restype = C.c_int
    lib.glqb_moe_plan_set_timing.argtypes = [vp, i32]
    lib.glqb_moe_plan_set_timing.restype = C.c_int
    lib.glqb_moe_plan_kernel_ms.argtypes = [vp, C.POINTER(C.c_double), C.POINTER(i32)]
    lib.glqb_moe_plan_kernel_ms.restype = C.c_int
    lib.glqb_moe_plan_destroy.argtypes = [vp]
    lib.glqb_moe_plan_destroy.restype = None
    lib.glqb_comm_create.argtypes = [i32, i32, i64, C.POINTER(vp)]
    lib.glqb_comm_create.restype = C.c_int
    lib.glqb_comm_handle.argtypes = [vp, vp, i32]
    lib.glqb_comm_handle.restype = C.c_int
    lib.glqb_comm_connect.argtypes = [vp, C.c_char_p, i32]
    lib.glqb_comm_connect.restype = C.c_int
    lib.glqb_comm_connect_local.argtypes = [vp, C.POINTER(vp)]
    lib.glqb_comm_connect_local.restype = C.c_int
    lib.glqb_comm_set_timeout_ms.argtypes = [vp, i32]
    lib.glqb_comm_set_timeout_ms.restype = C.c_int
    lib.glqb_comm_max_floats.argtypes = [vp]
    lib.glqb_comm_max_floats.restype = i64
    lib.glqb_comm_all_reduce.argtypes = [vp, vp, i64, vp]
    lib.glqb_comm_all_reduce.restype = C.c_int
    lib.glqb_comm_status.argtypes = [vp, C.POINTER(i32), i32]
    lib.glqb_comm_status.restype = C.c_int
    lib.glqb_comm_epoch.argtypes = [vp, C.POINTER(i32)]
    lib.glqb_comm_epoch.restype = C.c_int
    lib.glqb_comm_destroy.argtypes = [vp]
    lib.glqb_comm_destroy.restype = None
    lib.glqb_plan_set_comm.argtypes = [vp, vp]
    lib.glqb_plan_set_comm.restype = C.c_int
    lib.glqb_last_error.argtypes = []
    lib.glqb_last_error.restype = C.c_char_p
    lib.glqb_version.argtypes = []
    lib.glqb_version.restype = C.c_char_p
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = load().glqb_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"glq_b200: {what} failed (code {rc}): {msg}")
