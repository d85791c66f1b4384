"""The C restatement of the oracle (also the timed CPU baseline) against the numpy oracle and the
reference's golden outputs."""
import os

import numpy as np
import pytest

from oracle import c_oracle as CO
from oracle import glq_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_3inst_table_bit_exact(golden):
    g = golden("golden_trellis.npz")
    assert np.array_equal(CO.decode_3inst_table().view(np.uint16), g["table3inst_f16"].view(np.uint16))


@pytest.mark.parametrize("K", [1, 2, 3, 4])
def test_trellis_decode_bit_exact(golden, K):
    g = golden("golden_trellis.npz")
    for (m, n) in ((32, 64), (64, 192), (96, 128)):
        key = f"K{K}_m{m}_n{n}"
        dec = CO.trellis_decode(g[key + "_packed"], m, n, K)
        assert np.array_equal(dec.view(np.uint16), g[key + "_dec"].view(np.uint16))


@pytest.mark.parametrize("K2", [1, 2, 3, 4])
def test_trellis_two_stage_bit_exact(golden, K2):
    g = golden("golden_trellis.npz")
    key = f"rvq_K2_{K2}"
    dec = CO.trellis_decode_f32(g[key + "_p1"], 4, g[key + "_p2"], K2, float(g[key + "_inv"]), 64, 128)
    assert np.array_equal(dec.view(np.uint32), g[key + "_dec"].view(np.uint32))


def test_e8_decode_bit_exact(e8_table):
    packed = np.load(os.path.join(ROOT, "glq_b200", "data", "e8_shell_packed.npy"))
    rng = np.random.default_rng(0)
    m, n = 48, 128
    qs = [rng.integers(0, 65536, size=(m, n // 8), dtype=np.uint16).view(np.int16) for _ in range(4)]
    inv = [1 / 3.0, 1 / 9.0, 1 / 27.0]
    for ns in (1, 2, 3, 4):
        got = CO.e8_decode(qs[:ns], [packed] * ns, inv[:ns - 1], m, n)
        ref = O.e8_decode_nstage(qs[:ns], [e8_table] * ns, inv[:ns - 1])
        assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))


def test_fht_matches_reference(golden):
    g = golden("golden_misc.npz")
    np.testing.assert_allclose(CO.fht(g["fht_x"]), g["fht_y"], atol=1e-6)


@pytest.mark.parametrize("name", ["k2", "k4", "k4p2"])
def test_trellis_linear_matches_reference(golden, name):
    g = golden("golden_trellis_linear.npz")
    fin, fout, K, K2 = [int(v) for v in g[name + "_meta"]]
    y = CO.trellis_linear(g[name + "_x"], g[name + "_packed"], K, g[name + "_packed2"] if K2 else None, K2,
                          float(g[name + "_inv_resid_scale2"]), fout, fin, g[name + "_SU"], g[name + "_SV"],
                          float(g[name + "_Wscale"]), O.block_decompose(fin), O.block_decompose(fout))
    ref = g[name + "_y"]
    assert np.abs(y - ref).max() <= 2e-5 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("name", ["pow2_1s", "bd_2s_full", "bd_4s"])
def test_e8_linear_matches_reference(golden, name):
    g = golden("golden_e8_linear.npz")
    packed = np.load(os.path.join(ROOT, "glq_b200", "data", "e8_shell_packed.npy"))
    fin, fout, m_pad, n_pad, stages, bd, small = [int(v) for v in g[name + "_meta"]]
    qs = [g[f"{name}_Qidxs"], g[f"{name}_Qidxs2"], g[f"{name}_Qidxs3"], g[f"{name}_Qidxs4"]][:stages]
    inv = [float(g[f"{name}_inv_resid_scale"]), float(g[f"{name}_inv_resid_scale2"]),
           float(g[f"{name}_inv_resid_scale3"])][:stages - 1]
    y = CO.e8_linear(g[name + "_x"], qs, [packed] * stages, inv, m_pad, n_pad, g[name + "_SU"], g[name + "_SV"],
                     float(g[name + "_Wscale"]), list(g[name + "_blocks_n"]), list(g[name + "_blocks_m"]), fout)
    ref = g[name + "_y"]
    assert np.abs(y - ref).max() <= 2e-5 * max(1.0, np.abs(ref).max())
