"""``GLQLinear`` — the reference's ``E8RHTLinear`` (glq/quantized_linear.py:166-1265) served by libglq_b200.

Same constructor arguments, same buffer names and shapes (``Qidxs..Qidxs4``, ``inv_resid_scale..3``,
``trellis_packed``/``trellis_packed2``/``inv_resid_scale2``, ``SU``, ``SV``, ``Wscale``, ``bias``), so a
reference state dict loads unchanged; ``forward`` goes through the same operator functions the reference
calls by name.  There is no CPU path: on a CPU tensor ``forward`` raises.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import ops
from .plan import block_decompose


class GLQLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, bias: bool = False, block_diagonal: bool = False,
                 codebook_type: str = "e8_shell"):
        super().__init__()
        if codebook_type not in ("e8_shell", "trellis"):
            raise ValueError(f"glq_b200 serves e8_shell and trellis layers, not {codebook_type!r}")
        self.in_features, self.out_features = in_features, out_features
        self._is_trellis = codebook_type == "trellis"
        if self._is_trellis:
            block_diagonal = True
        if block_diagonal:                                   # glq/quantized_linear.py:217-222
            self.blocks_m, self.blocks_n = block_decompose(out_features), block_decompose(in_features)
            self.m_pad, self.n_pad = out_features, in_features
            if not self._is_trellis and self.n_pad % 8:
                raise ValueError("E8 layers need in_features to be a multiple of 8")
        else:                                                # legacy: pad to the next power of two (:224-228)
            self.m_pad = 1 << (out_features - 1).bit_length() if out_features > 0 else 1
            self.n_pad = 1 << (in_features - 1).bit_length() if in_features > 0 else 1
            self.blocks_m, self.blocks_n = [self.m_pad], [self.n_pad]
        self.block_diagonal = block_diagonal
        self.register_buffer("SU", torch.ones(self.m_pad, dtype=torch.float16))
        self.register_buffer("SV", torch.ones(self.n_pad, dtype=torch.float16))
        self.register_buffer("Wscale", torch.ones((), dtype=torch.float32))
        if self._is_trellis:
            self.register_buffer("trellis_packed", torch.zeros(0, dtype=torch.int16))
            self.register_buffer("trellis_packed2", torch.zeros(0, dtype=torch.int16))
            self.register_buffer("inv_resid_scale2", torch.zeros((), dtype=torch.float32))
            self.register_buffer("tlut", torch.zeros(0, dtype=torch.float16))
        else:
            shape = (self.m_pad, self.n_pad // 8)
            for name in ("Qidxs", "Qidxs2", "Qidxs3", "Qidxs4"):
                self.register_buffer(name, torch.zeros(shape, dtype=torch.int16))
            for name in ("inv_resid_scale", "inv_resid_scale2", "inv_resid_scale3"):
                self.register_buffer(name, torch.zeros((), dtype=torch.float32))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=torch.float16))
        else:
            self.bias = None
        self.codebook = None          # fp16 (65536, 8) tensor, or an object with .codebook_half
        self.codebook2 = None
        self._scalars = None          # cached host copies of the scalar buffers (no sync per forward)
        self._tables = {}             # converted codebooks per device

    # -- loading ---------------------------------------------------------------------------------------
    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        for name in ("trellis_packed", "trellis_packed2", "tlut"):      # sized by the checkpoint (:351-361)
            key = prefix + name
            if key in state_dict and hasattr(self, name):
                getattr(self, name).resize_(state_dict[key].shape)
        self._scalars = None
        return super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)

    def set_codebook(self, codebook, codebook2=None):
        """E8 layers: the shared codebook(s), as the reference's objects or as fp16 (entries, 8) tensors."""
        self.codebook, self.codebook2 = codebook, codebook2
        self._scalars = None
        self._tables = {}

    def _table(self, cb, device):
        """fp16 copy of a codebook on ``device``, converted once per (codebook, device) and kept: the packed
        table cache of the operator layer is keyed on the tensor's address."""
        t = getattr(cb, "codebook_half", cb)
        if t.device == device and t.dtype == torch.float16:
            return t
        key = (id(cb), str(device))
        hit = self._tables.get(key)
        if hit is None or hit[0] is not t:
            hit = (t, t.to(device=device, dtype=torch.float16))
            self._tables[key] = hit
        return hit[1]

    def _resolve(self):
        if self._scalars is None:
            s = {"wscale": float(self.Wscale.item())}
            if self._is_trellis:
                if self.tlut.numel():
                    raise NotImplementedError("HYB (tlut) trellis layers are not served; re-quantize with variant 3inst")
                s["has2"] = self.trellis_packed2.numel() > 0
                s["inv2"] = float(self.inv_resid_scale2.item()) if s["has2"] else 0.0
            else:
                inv = [float(getattr(self, n).item()) for n in ("inv_resid_scale", "inv_resid_scale2", "inv_resid_scale3")]
                n_stages = 1
                if self.codebook2 is not None and inv[0] != 0.0:       # glq/quantized_linear.py:434-451
                    n_stages = 2
                    if inv[1] != 0.0:
                        n_stages = 3
                        if inv[2] != 0.0:
                            n_stages = 4
                s["inv"], s["n_stages"] = inv, n_stages
            self._scalars = s
        return self._scalars

    # -- forward ---------------------------------------------------------------------------------------
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("glq_b200.GLQLinear has no CPU path")
        s = self._resolve()
        shape = x.shape
        x2d = x.reshape(-1, self.in_features)
        bn, bm = torch.tensor(self.blocks_n), torch.tensor(self.blocks_m)
        if self._is_trellis:
            if s["has2"]:
                y = ops.fused_linear_trellis_3inst_rvq2(x2d, self.SV, self.SU, self.trellis_packed, self.trellis_packed2,
                                                        bn, bm, None, None, s["wscale"], s["inv2"], self.in_features,
                                                        self.out_features, self.n_pad, self.m_pad)
            else:
                y = ops.fused_linear_trellis_3inst(x2d, self.SV, self.SU, self.trellis_packed, bn, bm, None, None,
                                                   s["wscale"], self.in_features, self.out_features, self.n_pad,
                                                   self.m_pad)
        else:
            if self.codebook is None:
                raise RuntimeError("set_codebook() has not been called")
            dev = x.device
            cb = self._table(self.codebook, dev)
            empty_i = torch.empty(0, dtype=torch.int16, device=dev)
            empty_h = torch.empty(0, dtype=torch.float16, device=dev)
            ns, inv = s["n_stages"], s["inv"]
            cb2 = self._table(self.codebook2, dev) if ns >= 2 else empty_h
            tail = (self.Qidxs2 if ns >= 2 else empty_i, cb2, inv[0] if ns >= 2 else 0.0,
                    self.Qidxs3 if ns >= 3 else empty_i, cb if ns >= 3 else empty_h, inv[1] if ns >= 3 else 0.0,
                    self.Qidxs4 if ns >= 4 else empty_i, cb if ns >= 4 else empty_h, inv[2] if ns >= 4 else 0.0)
            if self.block_diagonal:
                y = ops.fused_linear_block_diag(x2d, self.SV, self.SU, self.Qidxs, cb, s["wscale"], self.in_features,
                                                self.out_features, self.n_pad, self.m_pad, bn, bm, None, None, *tail)
            else:
                y = ops.fused_linear(x2d, self.SV, self.SU, self.Qidxs, cb, s["wscale"], self.in_features,
                                     self.out_features, self.n_pad, self.m_pad, self.n_pad.bit_length() - 1,
                                     self.m_pad.bit_length() - 1, *tail)
        if self.bias is not None:
            y = y + self.bias.unsqueeze(0).to(y.dtype)
        return y.reshape(*shape[:-1], self.out_features)

    # -- debugging -------------------------------------------------------------------------------------
    def dequantize_rotated(self) -> torch.Tensor:
        """fp32 (m_pad, n_pad) rotated-domain weights exactly as the kernels reconstruct them (unscaled)."""
        s = self._resolve()
        if self._is_trellis:
            if s["has2"]:
                return ops.decompress_trellis_3inst_rvq2(self.trellis_packed, self.trellis_packed2, s["inv2"],
                                                         self.m_pad, self.n_pad)
            return ops.glq_decompress_trellis_3inst_cuda(self.trellis_packed, self.m_pad, self.n_pad).float()
        dev = self.Qidxs.device
        ns = s["n_stages"]
        qs = [self.Qidxs, self.Qidxs2, self.Qidxs3, self.Qidxs4][:ns]
        cb = self._table(self.codebook, dev)
        cbs = [cb, self._table(self.codebook2, dev) if ns >= 2 else cb, cb, cb][:ns]
        return ops.dequant_e8(qs, cbs, s["inv"][:ns - 1])

    def dequantize(self) -> torch.Tensor:
        """Dense fp32 (out_features, in_features) weight: the rotated-domain weights the kernels reconstruct,
        scaled by Wscale and taken back through both Hadamard transforms (glq/quantized_linear.py:1237-1265),
        so that ``forward(x) == x @ dequantize().T`` up to rounding.  Every residual stage is included (the
        reference's helper stops after the second)."""
        W = self.dequantize_rotated().contiguous()                       # (m_pad, n_pad)
        dev = W.device
        bn, bm = self.blocks_n, self.blocks_m
        # columns: rows of W are "tokens" of the unfused transform, which gives SV * H_n(row) / sqrt(block)
        t = torch.empty_like(W)
        ops.output_rht_blocks(W, self.SV, t, self.n_pad, self.n_pad, bn)
        t2 = torch.empty(self.n_pad, self.m_pad, dtype=torch.float32, device=dev)
        ops.output_rht_blocks(t.t().contiguous(), self.SU, t2, self.m_pad, self.m_pad, bm)
        return (t2.t() * float(self.Wscale.item()))[:self.out_features, :self.in_features].contiguous()

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"m_pad={self.m_pad}, n_pad={self.n_pad}, trellis={self._is_trellis}")
