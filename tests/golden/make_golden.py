"""Generate the golden fixtures in this directory by running the REFERENCE (cnygaard/glq).

Usage (only where the reference package is importable; it is not needed to run tests):

    TORCHDYNAMO_DISABLE=1 PYTHONPATH=<path-to-reference> python tests/golden/make_golden.py

Writes ``golden_trellis.npz``, ``golden_e8_linear.npz``, ``golden_trellis_linear.npz``
and ``golden_misc.npz`` next to this file.  Every array is an input to, or an output of,
the reference's own CPU code (``glq.trellis.decode_layer``, ``E8RHTLinear.forward``,
``glq.hadamard``), so the oracle and the CUDA kernels are checked against the reference
itself and not against a restatement of it.
"""
import hashlib
import os
import sys

os.environ.setdefault("TORCHDYNAMO_DISABLE", "1")

import numpy as np
import torch

from glq.codebook import E8ShellCodebook
from glq.hadamard import _block_decompose, _pytorch_fht, block_diagonal_fht
from glq.quantized_linear import E8RHTLinear
from glq.trellis import (TrellisCodebook, _INV_PERMUTE, _PERMUTE, decode_3inst, decode_layer,
                         decode_layer_nstage)

HERE = os.path.dirname(os.path.abspath(__file__))


def signs(rng, n):
    return (rng.integers(0, 2, size=n) * 2 - 1).astype(np.float16)


def gen_trellis():
    rng = np.random.default_rng(1234)
    out = {}
    tab = decode_3inst(torch.arange(65536)).numpy()
    out["table3inst_f16"] = tab.astype(np.float16)
    assert np.array_equal(out["table3inst_f16"].astype(np.float32), tab)
    for K in (1, 2, 3, 4):
        cb = TrellisCodebook(variant="3inst", K=K)
        for (m, n) in ((32, 64), (64, 192), (96, 128)):
            packed = rng.integers(0, 65536, size=((m // 16) * (n // 16), 16 * K),
                                  dtype=np.uint16).view(np.int16)
            dec = decode_layer(cb.cb, torch.from_numpy(packed.copy()), m, n, True).numpy()
            key = f"K{K}_m{m}_n{n}"
            out[key + "_packed"] = packed
            out[key + "_dec"] = dec.astype(np.float16)
            assert np.array_equal(out[key + "_dec"].astype(np.float32), dec)
    # stacked two-stage decode (4 + K2), fp32
    m, n = 64, 128
    for K2 in (1, 2, 3, 4):
        cb1 = TrellisCodebook(variant="3inst", K=4)
        cb2 = TrellisCodebook(variant="3inst", K=K2)
        p1 = rng.integers(0, 65536, size=((m // 16) * (n // 16), 64), dtype=np.uint16).view(np.int16)
        p2 = rng.integers(0, 65536, size=((m // 16) * (n // 16), 16 * K2), dtype=np.uint16).view(np.int16)
        inv = float(np.float32(0.1 + 0.05 * K2))
        dec = decode_layer_nstage([cb1.cb, cb2.cb], [torch.from_numpy(p1.copy()), torch.from_numpy(p2.copy())],
                                  [1.0, inv], m, n, True).numpy()
        key = f"rvq_K2_{K2}"
        out[key + "_p1"] = p1
        out[key + "_p2"] = p2
        out[key + "_inv"] = np.float32(inv)
        out[key + "_dec"] = dec.astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "golden_trellis.npz"), **out)


def gen_e8_linear(cb):
    rng = np.random.default_rng(4321)
    out = {}
    small = cb.make_small(256)
    cases = [
        # name, in, out, block_diag, stages, second-stage table
        ("pow2_1s", 48, 32, False, 1, None),
        ("pow2_2s_small", 64, 64, False, 2, "small"),
        ("bd_1s", 576, 160, True, 1, None),
        ("bd_2s_full", 320, 96, True, 2, "full"),
        ("bd_3s", 192, 96, True, 3, "full"),
        ("bd_4s", 192, 160, True, 4, "full"),
    ]
    for name, fin, fout, bd, stages, cb2kind in cases:
        layer = E8RHTLinear(fin, fout, block_diagonal=bd)
        m_pad, n_pad = layer.m_pad, layer.n_pad
        hi = 65536
        layer.Qidxs.copy_(torch.from_numpy(
            rng.integers(0, hi, size=(m_pad, n_pad // 8), dtype=np.uint16).view(np.int16).copy()))
        layer.SU.copy_(torch.from_numpy(signs(rng, m_pad)))
        layer.SV.copy_(torch.from_numpy(signs(rng, n_pad)))
        layer.Wscale.fill_(float(rng.uniform(0.5, 1.5) * 0.02))
        cb2 = None
        if stages >= 2:
            hi2 = 256 if cb2kind == "small" else 65536
            layer.Qidxs2.copy_(torch.from_numpy(
                rng.integers(0, hi2, size=(m_pad, n_pad // 8), dtype=np.uint16).view(np.int16).copy()))
            layer.inv_resid_scale.fill_(1.0 / 3.0)
            cb2 = small if cb2kind == "small" else cb
        if stages >= 3:
            layer.Qidxs3.copy_(torch.from_numpy(
                rng.integers(0, 65536, size=(m_pad, n_pad // 8), dtype=np.uint16).view(np.int16).copy()))
            layer.inv_resid_scale2.fill_(1.0 / 9.0)
        if stages >= 4:
            layer.Qidxs4.copy_(torch.from_numpy(
                rng.integers(0, 65536, size=(m_pad, n_pad // 8), dtype=np.uint16).view(np.int16).copy()))
            layer.inv_resid_scale3.fill_(1.0 / 27.0)
        layer.set_codebook(cb, codebook2=cb2)
        assert layer._n_stages == stages, (name, layer._n_stages)
        x = torch.from_numpy(rng.standard_normal((5, fin)).astype(np.float32))
        with torch.no_grad():
            y = layer(x).numpy()
        out[name + "_meta"] = np.array([fin, fout, m_pad, n_pad, stages, int(bd),
                                        0 if cb2kind != "small" else 256], dtype=np.int64)
        out[name + "_blocks_n"] = np.array(layer.blocks_n, dtype=np.int64)
        out[name + "_blocks_m"] = np.array(layer.blocks_m, dtype=np.int64)
        for k in ("Qidxs", "Qidxs2", "Qidxs3", "Qidxs4", "SU", "SV", "Wscale",
                  "inv_resid_scale", "inv_resid_scale2", "inv_resid_scale3"):
            out[f"{name}_{k}"] = getattr(layer, k).numpy()
        out[name + "_x"] = x.numpy()
        out[name + "_y"] = y
        if stages <= 2 and not bd:
            out[name + "_dequant"] = layer.dequantize().numpy()
    np.savez_compressed(os.path.join(HERE, "golden_e8_linear.npz"), **out)


def gen_trellis_linear():
    rng = np.random.default_rng(999)
    out = {}
    cases = [("k2", 192, 96, 2, 0), ("k3", 128, 64, 3, 0), ("k4", 320, 160, 4, 0),
             ("k4p2", 192, 96, 4, 2), ("k4p4", 128, 128, 4, 4)]
    for name, fin, fout, K, K2 in cases:
        layer = E8RHTLinear(fin, fout, codebook_type="trellis")
        m, n = layer.m_pad, layer.n_pad
        p1 = rng.integers(0, 65536, size=((m // 16) * (n // 16), 16 * K), dtype=np.uint16).view(np.int16)
        layer.trellis_packed.resize_(p1.shape).copy_(torch.from_numpy(p1.copy()))
        cb1 = TrellisCodebook(variant="3inst", K=K)
        cb2 = None
        if K2:
            p2 = rng.integers(0, 65536, size=((m // 16) * (n // 16), 16 * K2), dtype=np.uint16).view(np.int16)
            layer.trellis_packed2.resize_(p2.shape).copy_(torch.from_numpy(p2.copy()))
            layer.inv_resid_scale2.fill_(0.21)
            cb2 = TrellisCodebook(variant="3inst", K=K2)
            out[name + "_packed2"] = p2
        layer.SU.copy_(torch.from_numpy(signs(rng, m)))
        layer.SV.copy_(torch.from_numpy(signs(rng, n)))
        layer.Wscale.fill_(float(rng.uniform(0.5, 1.5) * 0.02))
        layer.set_codebook(cb1, codebook2=cb2)
        # the pure-torch path wants the inner bitshift codebooks
        layer.codebook = cb1.cb
        layer.codebook2 = cb2.cb if cb2 is not None else None
        layer._ensure_trellis_codebook_device = lambda dev: None
        layer._ensure_trellis_codebook2_device = lambda dev: None
        x = torch.from_numpy(rng.standard_normal((3, fin)).astype(np.float32))
        with torch.no_grad():
            y = layer(x).numpy()
        out[name + "_meta"] = np.array([fin, fout, K, K2], dtype=np.int64)
        out[name + "_packed"] = p1
        out[name + "_SU"] = layer.SU.numpy()
        out[name + "_SV"] = layer.SV.numpy()
        out[name + "_Wscale"] = layer.Wscale.numpy()
        out[name + "_inv_resid_scale2"] = layer.inv_resid_scale2.numpy()
        out[name + "_x"] = x.numpy()
        out[name + "_y"] = y
    np.savez_compressed(os.path.join(HERE, "golden_trellis_linear.npz"), **out)


def gen_misc(cb):
    rng = np.random.default_rng(7)
    out = {}
    x = torch.from_numpy(rng.standard_normal((3, 64)).astype(np.float32))
    out["fht_x"] = x.numpy().copy()
    out["fht_y"] = _pytorch_fht(x.clone()).numpy()
    xb = torch.from_numpy(rng.standard_normal((2, 2688)).astype(np.float32))
    out["bd_x"] = xb.numpy().copy()
    out["bd_blocks"] = np.array(_block_decompose(2688), dtype=np.int64)
    out["bd_y"] = block_diagonal_fht(xb.clone(), _block_decompose(2688)).numpy()
    for n in (2688, 4096, 11008, 5376, 21504, 14336, 1536, 768):
        out[f"decomp_{n}"] = np.array(_block_decompose(n), dtype=np.int64)
    out["permute"] = _PERMUTE.numpy()
    out["inv_permute"] = _INV_PERMUTE.numpy()
    tab = cb.codebook.numpy()
    out["e8_sha256"] = np.frombuffer(hashlib.sha256(tab.tobytes()).digest(), dtype=np.uint8)
    out["e8_rows_sample_idx"] = np.array([0, 1, 2, 240, 241, 2400, 2401, 9120, 9121, 26640, 26641,
                                          56880, 56881, 65535], dtype=np.int64)
    out["e8_rows_sample"] = tab[out["e8_rows_sample_idx"]]
    out["e8_opt_scale"] = np.float64(cb.opt_scale)
    out["e8_resid_scale"] = np.float64(cb.resid_scale)
    np.savez_compressed(os.path.join(HERE, "golden_misc.npz"), **out)


if __name__ == "__main__":
    cb = E8ShellCodebook.build(device="cpu", verbose=False)
    gen_trellis()
    gen_e8_linear(cb)
    gen_trellis_linear()
    gen_misc(cb)
    print("golden fixtures written to", HERE)
