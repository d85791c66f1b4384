"""Put libglq_b200 behind the reference's entry points without editing reference files.

``install()`` does what INTEGRATION.md describes: it makes ``glq.inference_kernel`` believe its
extension is already loaded (the loader returns early, glq/inference_kernel.py:228-230) and hands it
this package's operator module, whose functions carry the names the reference looks up with
``hasattr`` (glq/quantized_linear.py:873-896, 1079-1120).  When the reference's vLLM plugin is
importable, its op registration is marked done (glq_vllm/custom_ops.py:15, 41-44) and the same
functions are registered under ``torch.ops.glq`` so ``torch.compile`` sees single opaque nodes.
"""
from __future__ import annotations

import importlib
import sys

from . import ops

# names the reference probes on its extension module (glq/csrc/glq_bindings.cpp:334-550) that this
# library serves; anything else stays absent so that the reference's own capability checks refuse it
SERVED = [
    "glq_fused_linear_cuda", "glq_fused_linear_block_diag_cuda", "glq_fused_linear_trellis_3inst_cuda",
    "glq_fused_linear_trellis_3inst_rvq2_cuda", "glq_fused_linear_trellis_3inst_yrht_cuda",
    "glq_fused_linear_trellis_3inst_yrht_rvq2_cuda", "glq_output_rht_shards_cuda", "glq_dequant_matvec_cuda",
    "glq_dequant_matmul_cuda", "glq_input_rht_cuda", "glq_output_rht_cuda", "glq_trellis_kernel_supported",
    "glq_decompress_trellis_3inst_cuda", "glq_fused_moe_trellis_3inst_cuda",
]

OP_SCHEMAS = {   # torch.ops.glq name -> (schema, python function); schemas from glq_vllm/custom_ops.py
    "fused_linear_trellis_3inst": (
        "fused_linear_trellis_3inst(Tensor x, Tensor sv, Tensor su, Tensor trellis_packed, Tensor blocks_n, "
        "Tensor blocks_m, Tensor blocks_n_meta, Tensor blocks_m_meta, float wscale, int in_features, "
        "int out_features, int n_pad, int m_pad) -> Tensor", ops.fused_linear_trellis_3inst),
    "fused_linear_trellis_3inst_rvq2": (
        "fused_linear_trellis_3inst_rvq2(Tensor x, Tensor sv, Tensor su, Tensor trellis_packed, "
        "Tensor trellis_packed2, Tensor blocks_n, Tensor blocks_m, Tensor blocks_n_meta, Tensor blocks_m_meta, "
        "float wscale, float inv_resid_scale2, int in_features, int out_features, int n_pad, int m_pad) -> Tensor",
        ops.fused_linear_trellis_3inst_rvq2),
}


class _ExtensionProxy:
    """Stands where the reference expects its pybind module: only the served names exist."""

    def __init__(self):
        for name in SERVED:
            setattr(self, name, getattr(ops, name))


def install(register_torch_ops: bool = True):
    """Returns the proxy installed as ``glq.inference_kernel._glq_cuda``.  Raises ImportError when the
    reference package is not importable (then use ``glq_b200.ops`` / ``GLQLinear`` directly)."""
    ik = importlib.import_module("glq.inference_kernel")
    proxy = _ExtensionProxy()
    ik._glq_cuda = proxy
    ik._cuda_ext_available = True
    if register_torch_ops:
        co = sys.modules.get("glq_vllm.custom_ops")
        if co is None:
            try:
                co = importlib.import_module("glq_vllm.custom_ops")
            except Exception:
                co = None
        if co is not None and not getattr(co, "_registered", False):
            co._registered = True
            lib = getattr(co, "_glq_lib", None)
            if lib is not None:
                for name, (schema, fn) in OP_SCHEMAS.items():
                    try:
                        lib.define(schema)
                        lib.impl(name, fn, "CUDA")
                    except RuntimeError:
                        pass          # already defined by another installer
    return proxy
