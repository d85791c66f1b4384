"""Put libglq_b200 behind the reference's entry points without editing reference files.

Two lookups have to find this library's operators:

* ``glq.inference_kernel._glq_cuda`` — the reference's extension module.  ``install()`` makes the loader
  believe the extension is already loaded (it returns early, glq/inference_kernel.py:228-230) and hands it
  a proxy whose attributes carry the names the reference probes with ``hasattr``
  (glq/quantized_linear.py:873-896, 1079-1120).
* ``torch.ops.glq.*`` — what the vLLM plugin calls (glq_vllm/linear_method.py:451, 466-522, 662-710;
  glq_vllm/fused_moe_method.py:709-738, 913-1010).  ``register_torch_ops()`` defines every served op with
  the reference's schema string (glq_vllm/custom_ops.py:58-428), implements it for the CUDA dispatch key
  with the function of the same name in :mod:`glq_b200.ops`, and registers a fake (meta) implementation
  that only computes the output's shape, dtype and device, so ``torch.compile`` and CUDA-graph capture see
  each GLQ op as one opaque node.  The reference's own registration is then marked as done
  (glq_vllm/custom_ops.py:15, 41-44) so that it does not try to define the same names again.

Ops of formats this library does not serve (HYB trellis, E8P, the packed 2-bpw variants, the KV-cache
gathers) are deliberately left undefined: the reference's capability checks then refuse or fall back.
"""
from __future__ import annotations

import importlib
import sys

import torch

from . import ops

# names the reference probes on its extension module (glq/csrc/glq_bindings.cpp:334-550) that this
# library serves; anything else stays absent so that the reference's own capability checks refuse it
SERVED = [
    "glq_fused_linear_cuda", "glq_fused_linear_block_diag_cuda", "glq_fused_linear_trellis_3inst_cuda",
    "glq_fused_linear_trellis_3inst_rvq2_cuda", "glq_fused_linear_trellis_3inst_yrht_cuda",
    "glq_fused_linear_trellis_3inst_yrht_rvq2_cuda", "glq_output_rht_shards_cuda", "glq_dequant_matvec_cuda",
    "glq_dequant_matmul_cuda", "glq_input_rht_cuda", "glq_output_rht_cuda", "glq_trellis_kernel_supported",
    "glq_decompress_trellis_3inst_cuda", "glq_fused_moe_trellis_3inst_cuda", "glq_fused_moe_grouped_gemm_cuda",
    "glq_fused_moe_block_diag_cuda",
]

_E8_TAIL = ("Tensor qidxs2, Tensor codebook2, float inv_resid_scale, "
            "Tensor qidxs3, Tensor codebook3, float inv_resid_scale2, "
            "Tensor qidxs4, Tensor codebook4, float inv_resid_scale3")
_BLOCKS = "Tensor blocks_n, Tensor blocks_m, Tensor blocks_n_meta, Tensor blocks_m_meta"
_MOE_E8_ARGS = (
    "(Tensor x, Tensor topk_ids, Tensor topk_weights, "
    "Tensor w13_Qidxs, Tensor w13_SU, Tensor w13_SV, Tensor w13_Wscale, Tensor w13_Qidxs2, Tensor w13_inv_rs, "
    "Tensor w2_Qidxs, Tensor w2_SU, Tensor w2_SV, Tensor w2_Wscale, Tensor w2_Qidxs2, Tensor w2_inv_rs, "
    "Tensor codebook, Tensor codebook2, "
    "int hidden_size, int intermediate_size, int w13_out_features, "
    "int n_pad_w13, int m_pad_w13, int n_pad_w2, int m_pad_w2, "
    "Tensor blocks_n_w13, Tensor blocks_m_w13, Tensor blocks_n_w13_meta, Tensor blocks_m_w13_meta, "
    "Tensor blocks_n_w2, Tensor blocks_m_w2, Tensor blocks_n_w2_meta, Tensor blocks_m_w2_meta, "
    "int activation_type, "
    "Tensor w13_Qidxs3, Tensor w13_inv_rs2, Tensor w2_Qidxs3, Tensor w2_inv_rs2, Tensor codebook3) -> Tensor")
_MOE_TRELLIS_ARGS = (
    "(Tensor x, Tensor topk_ids, Tensor topk_weights, "
    "Tensor w13_trellis_packed, Tensor w13_trellis_packed2, Tensor w13_SU, Tensor w13_SV, Tensor w13_Wscale, "
    "Tensor w13_inv_resid_scale2, "
    "Tensor w2_trellis_packed, Tensor w2_trellis_packed2, Tensor w2_SU, Tensor w2_SV, Tensor w2_Wscale, "
    "Tensor w2_inv_resid_scale2, "
    "int hidden_size, int intermediate_size, int w13_out_features, "
    "int n_pad_w13, int m_pad_w13, int n_pad_w2, int m_pad_w2, "
    "Tensor blocks_n_w13, Tensor blocks_m_w13, Tensor blocks_n_w13_meta, Tensor blocks_m_w13_meta, "
    "Tensor blocks_n_w2, Tensor blocks_m_w2, Tensor blocks_n_w2_meta, Tensor blocks_m_w2_meta, "
    "int activation_type) -> Tensor")


# ---- fake (meta) implementations: shape, dtype and device of the result, nothing else -----------------
# The results follow the activation dtype (the reference's kernels are fp16-only and its callers cast to
# fp16 first, so for them this is fp16 as in glq_vllm/custom_ops.py:433-739).
def _rows_by(x, cols):
    return torch.empty((x.shape[0], int(cols)), dtype=x.dtype, device=x.device)


def _fake_dequant_matvec(x, qidxs, codebook, wscale, qidxs2, codebook2, inv_resid_scale, codebook_abs):
    return torch.empty(qidxs.shape[0], dtype=torch.float32, device=x.device)


def _fake_dequant_matmul(x, qidxs, codebook, wscale, qidxs2, codebook2, inv_resid_scale, codebook_abs,
                         qidxs3, codebook3, inv_resid_scale2, qidxs4, codebook4, inv_resid_scale3):
    return torch.empty((x.shape[0], qidxs.shape[0]), dtype=torch.float32, device=x.device)


def _fake_input_rht(x, sv, out, in_features, stride_x, rsqrt_n, n_pad, log_n):
    return None


def _fake_output_rht(y_rht, su, out, out_features, m_pad, log_m, rsqrt_m):
    return None


def _fake_fused_linear(x, sv, su, qidxs, codebook, wscale, in_features, out_features, n_pad, m_pad, log_n, log_m,
                       qidxs2, codebook2, inv_resid_scale, qidxs3, codebook3, inv_resid_scale2,
                       qidxs4, codebook4, inv_resid_scale3):
    return _rows_by(x, out_features)


def _fake_fused_linear_block_diag(x, sv, su, qidxs, codebook, wscale, in_features, out_features, n_pad, m_pad,
                                  blocks_n, blocks_m, blocks_n_meta, blocks_m_meta,
                                  qidxs2, codebook2, inv_resid_scale, qidxs3, codebook3, inv_resid_scale2,
                                  qidxs4, codebook4, inv_resid_scale3):
    return _rows_by(x, out_features)


def _fake_trellis(x, sv, su, trellis_packed, blocks_n, blocks_m, blocks_n_meta, blocks_m_meta, wscale,
                  in_features, out_features, n_pad, m_pad):
    return _rows_by(x, out_features)


def _fake_trellis_rvq2(x, sv, su, trellis_packed, trellis_packed2, blocks_n, blocks_m, blocks_n_meta,
                       blocks_m_meta, wscale, inv_resid_scale2, in_features, out_features, n_pad, m_pad):
    return _rows_by(x, out_features)


def _fake_trellis_yrht(x, sv, trellis_packed, blocks_n, blocks_n_meta, wscale, in_features, n_pad, m_pad,
                       y_rht_out, col):
    return None


def _fake_trellis_yrht_rvq2(x, sv, trellis_packed, trellis_packed2, blocks_n, blocks_n_meta, wscale,
                            inv_resid_scale2, in_features, n_pad, m_pad, y_rht_out, col):
    return None


def _fake_output_rht_shards(y_rht, su, y, out_features, shard_meta, max_bs):
    return None


def _fake_moe(x, *args):
    return torch.empty_like(x)


# torch.ops.glq name -> (schema without the name, implementation, fake)
OPS = {
    "dequant_matvec": ("(Tensor x, Tensor qidxs, Tensor codebook, float wscale, Tensor qidxs2, Tensor codebook2, "
                       "float inv_resid_scale, Tensor codebook_abs) -> Tensor", ops.dequant_matvec, _fake_dequant_matvec),
    "dequant_matmul": ("(Tensor x, Tensor qidxs, Tensor codebook, float wscale, Tensor qidxs2, Tensor codebook2, "
                       "float inv_resid_scale, Tensor codebook_abs, Tensor qidxs3, Tensor codebook3, "
                       "float inv_resid_scale2, Tensor qidxs4, Tensor codebook4, float inv_resid_scale3) -> Tensor",
                       ops.dequant_matmul, _fake_dequant_matmul),
    "input_rht": ("(Tensor x, Tensor sv, Tensor(a!) out, int in_features, int stride_x, float rsqrt_n, int n_pad, "
                  "int log_n) -> ()", ops.input_rht, _fake_input_rht),
    "output_rht": ("(Tensor y_rht, Tensor su, Tensor(a!) out, int out_features, int m_pad, int log_m, "
                   "float rsqrt_m) -> ()", ops.output_rht, _fake_output_rht),
    "fused_linear": ("(Tensor x, Tensor sv, Tensor su, Tensor qidxs, Tensor codebook, float wscale, "
                     "int in_features, int out_features, int n_pad, int m_pad, int log_n, int log_m, "
                     + _E8_TAIL + ") -> Tensor", ops.fused_linear, _fake_fused_linear),
    "fused_linear_block_diag": ("(Tensor x, Tensor sv, Tensor su, Tensor qidxs, Tensor codebook, float wscale, "
                                "int in_features, int out_features, int n_pad, int m_pad, " + _BLOCKS + ", "
                                + _E8_TAIL + ") -> Tensor", ops.fused_linear_block_diag, _fake_fused_linear_block_diag),
    "fused_linear_trellis_3inst": ("(Tensor x, Tensor sv, Tensor su, Tensor trellis_packed, " + _BLOCKS + ", "
                                   "float wscale, int in_features, int out_features, int n_pad, int m_pad) -> Tensor",
                                   ops.fused_linear_trellis_3inst, _fake_trellis),
    "fused_linear_trellis_3inst_rvq2": ("(Tensor x, Tensor sv, Tensor su, Tensor trellis_packed, "
                                        "Tensor trellis_packed2, " + _BLOCKS + ", float wscale, "
                                        "float inv_resid_scale2, int in_features, int out_features, int n_pad, "
                                        "int m_pad) -> Tensor", ops.fused_linear_trellis_3inst_rvq2, _fake_trellis_rvq2),
    "fused_linear_trellis_3inst_yrht": ("(Tensor x, Tensor sv, Tensor trellis_packed, Tensor blocks_n, "
                                        "Tensor blocks_n_meta, float wscale, int in_features, int n_pad, int m_pad, "
                                        "Tensor(a!) y_rht_out, int col) -> ()",
                                        ops.fused_linear_trellis_3inst_yrht, _fake_trellis_yrht),
    "fused_linear_trellis_3inst_yrht_rvq2": ("(Tensor x, Tensor sv, Tensor trellis_packed, Tensor trellis_packed2, "
                                             "Tensor blocks_n, Tensor blocks_n_meta, float wscale, "
                                             "float inv_resid_scale2, int in_features, int n_pad, int m_pad, "
                                             "Tensor(a!) y_rht_out, int col) -> ()",
                                             ops.fused_linear_trellis_3inst_yrht_rvq2, _fake_trellis_yrht_rvq2),
    "output_rht_shards": ("(Tensor y_rht, Tensor su, Tensor(a!) y, int out_features, Tensor shard_meta, "
                          "int max_bs) -> ()", ops.output_rht_shards, _fake_output_rht_shards),
    "fused_moe_trellis_3inst": (_MOE_TRELLIS_ARGS, ops.fused_moe_trellis_3inst, _fake_moe),
    "fused_moe_grouped_gemm": (_MOE_E8_ARGS, ops.fused_moe_grouped_gemm, _fake_moe),
    "fused_moe_block_diag": (_MOE_E8_ARGS, ops.fused_moe_block_diag, _fake_moe),
}

_LIBRARY = None           # keeps the registrations alive for the life of the process
_REGISTERED: list = []


class _ExtensionProxy:
    """Stands where the reference expects its pybind module: only the served names exist."""

    def __init__(self):
        for name in SERVED:
            setattr(self, name, getattr(ops, name))


def register_torch_ops(dispatch_key: str = "CUDA") -> list:
    """Define, implement and give a fake to every op of ``OPS`` under ``torch.ops.glq``.  Idempotent; an op
    that another component has already defined is left alone.  Returns the names registered by this call
    or an earlier one."""
    global _LIBRARY
    if _LIBRARY is None:
        _LIBRARY = torch.library.Library("glq", "FRAGMENT")
    for name, (schema, impl, fake) in OPS.items():
        if name in _REGISTERED:
            continue
        try:
            _LIBRARY.define(name + schema)
        except RuntimeError:
            continue                  # defined elsewhere (for instance by the reference's own extension)
        _LIBRARY.impl(name, impl, dispatch_key)
        torch.library.register_fake("glq::" + name, fake, lib=_LIBRARY)
        _REGISTERED.append(name)
    return list(_REGISTERED)


def install(register_ops: bool = True):
    """Returns the proxy installed as ``glq.inference_kernel._glq_cuda``.  Raises ImportError when the
    reference package is not importable (then use ``glq_b200.ops`` / ``GLQLinear`` directly, or only
    ``register_torch_ops()``)."""
    ik = importlib.import_module("glq.inference_kernel")
    proxy = _ExtensionProxy()
    ik._glq_cuda = proxy
    ik._cuda_ext_available = True
    if register_ops:
        register_torch_ops()
        co = sys.modules.get("glq_vllm.custom_ops")
        if co is None:
            try:
                co = importlib.import_module("glq_vllm.custom_ops")
            except Exception:
                co = None
        if co is not None:
            co._registered = True      # every op it would define for the served formats now exists
    return proxy
