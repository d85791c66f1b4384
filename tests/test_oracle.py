"""The CPU oracle against the reference's own outputs (tests/golden) and known answers."""
import hashlib

import numpy as np
import pytest

from oracle import glq_oracle as O


def test_3inst_table_matches_reference(golden):
    g = golden("golden_trellis.npz")
    assert np.array_equal(O.table_3inst().view(np.uint16), g["table3inst_f16"].view(np.uint16))


def test_3inst_values_are_two_fp16_halves():
    # known-answer: state 0 -> h = ADD; halves decoded by hand
    h = O.ADD_3INST
    r = (h & O.MASK_3INST) ^ O.XOR_3INST
    hi = np.array([r >> 16], dtype=np.uint16).view(np.float16)
    lo = np.array([r & 0xFFFF], dtype=np.uint16).view(np.float16)
    assert O.decode_3inst(np.array([0]))[0] == (hi + lo)[0]


@pytest.mark.parametrize("K", [1, 2, 3, 4])
@pytest.mark.parametrize("shape", [(32, 64), (64, 192), (96, 128)])
def test_trellis_decode_layer_bit_exact(golden, K, shape):
    g = golden("golden_trellis.npz")
    m, n = shape
    key = f"K{K}_m{m}_n{n}"
    dec = O.trellis_decode_layer(g[key + "_packed"], m, n, K)
    assert np.array_equal(dec.view(np.uint16), g[key + "_dec"].view(np.uint16))


@pytest.mark.parametrize("K2", [1, 2, 3, 4])
def test_trellis_two_stage_decode_bit_exact(golden, K2):
    g = golden("golden_trellis.npz")
    key = f"rvq_K2_{K2}"
    dec = O.trellis_decode_layer_nstage([g[key + "_p1"], g[key + "_p2"]], [4, K2],
                                        [1.0, float(g[key + "_inv"])], 64, 128)
    assert np.array_equal(dec.view(np.uint32), g[key + "_dec"].view(np.uint32))


@pytest.mark.parametrize("K", [1, 2, 3, 4])
def test_trellis_pack_unpack_round_trip(K):
    rng = np.random.default_rng(K)
    m, n = 64, 96
    packed = rng.integers(0, 65536, size=((m // 16) * (n // 16), 16 * K), dtype=np.uint16).view(np.int16)
    st = O.trellis_states(packed, m, n, K)
    assert np.array_equal(O.trellis_pack_states(st, K), packed)


def test_permutation_known_answers(golden):
    g = golden("golden_misc.npz")
    perm, inv = g["permute"], g["inv_permute"]
    assert np.array_equal(inv[perm], np.arange(256))
    # position maps used by the oracle are the same permutation written per (lane, j)
    rows, cols = O._TILE_ROW, O._TILE_COL
    flat = (rows * 16 + cols).reshape(-1)           # kernel order p -> natural index
    assert np.array_equal(flat, perm)


def test_e8_table_fingerprint_and_structure(golden, e8_table):
    g = golden("golden_misc.npz")
    digest = np.frombuffer(hashlib.sha256(e8_table.astype(np.float32).tobytes()).digest(), dtype=np.uint8)
    assert np.array_equal(digest, g["e8_sha256"])
    assert hashlib.sha256(e8_table.astype(np.float32).tobytes()).hexdigest().startswith("c46821e43e5a573c")
    assert np.array_equal(e8_table[g["e8_rows_sample_idx"]], g["e8_rows_sample"])
    n2 = (e8_table.astype(np.float64) ** 2).sum(1)
    assert np.all(np.diff(n2) >= 0)
    vals, counts = np.unique(n2, return_counts=True)
    assert list(vals) == [0, 2, 4, 6, 8, 10, 12]
    assert list(counts[:6]) == O.E8_SHELL_SIZES[:6] and counts[6] == 65536 - sum(O.E8_SHELL_SIZES[:6])
    # every row is an E8 point: all-integer or all-half-integer, even coordinate sum
    two = np.rint(e8_table * 2).astype(np.int64)
    par = two % 2
    assert np.all((par == par[:, :1]).all(1))
    assert np.all(two.sum(1) % 4 == 0)
    assert len({r.tobytes() for r in two}) == 65536
    assert np.array_equal(O.e8_unpack_table(O.e8_pack_table(e8_table)), e8_table)


def test_e8_shells_0_to_5_are_complete(e8_table):
    """Independent enumeration: every E8 point with squared norm <= 10 is in the table."""
    import itertools
    have = {tuple(r) for r in np.rint(e8_table[:56881] * 2).astype(np.int64)}
    # integer points (doubled coords even) with sum even, |v|^2<=10 -> doubled norm <= 40
    count = 0
    def rec(prefix, budget, vals):
        nonlocal count
        if len(prefix) == 8:
            if sum(prefix) % 4 == 0:
                assert tuple(prefix) in have
                count += 1
            return
        for v in vals:
            if v * v <= budget:
                rec(prefix + [v], budget - v * v, vals)
    rec([], 40, [-6, -4, -2, 0, 2, 4, 6])
    rec([], 40, [-5, -3, -1, 1, 3, 5])
    assert count == 56881


def test_fht_known_answers(golden):
    g = golden("golden_misc.npz")
    np.testing.assert_allclose(O.fht(g["fht_x"]), g["fht_y"], rtol=0, atol=1e-6)
    np.testing.assert_allclose(O.fht(O.fht(g["fht_x"])), g["fht_x"], atol=1e-5)     # involution
    e0 = np.zeros(8, dtype=np.float32); e0[0] = 1
    np.testing.assert_allclose(O.fht(e0), np.full(8, 1 / np.sqrt(8)), atol=1e-7)
    np.testing.assert_allclose(O.block_diag_fht(g["bd_x"], list(g["bd_blocks"])), g["bd_y"], atol=2e-6)
    for n in (2688, 4096, 11008, 5376, 21504, 14336, 1536, 768):
        assert O.block_decompose(n) == list(g[f"decomp_{n}"])
    assert O.block_decompose(2688) == [2048, 512, 128]


E8_CASES = ["pow2_1s", "pow2_2s_small", "bd_1s", "bd_2s_full", "bd_3s", "bd_4s"]


def _e8_rot_weight(g, name, e8_table):
    fin, fout, m_pad, n_pad, stages, bd, small = [int(v) for v in g[name + "_meta"]]
    qs = [g[f"{name}_Qidxs"], g[f"{name}_Qidxs2"], g[f"{name}_Qidxs3"], g[f"{name}_Qidxs4"]][:stages]
    tabs = [e8_table, e8_table[:256] if small else e8_table, e8_table, e8_table][:stages]
    inv = [float(g[f"{name}_inv_resid_scale"]), float(g[f"{name}_inv_resid_scale2"]),
           float(g[f"{name}_inv_resid_scale3"])][:stages - 1]
    return O.e8_decode_nstage(qs, tabs, inv), (fin, fout, m_pad, n_pad)


@pytest.mark.parametrize("name", E8_CASES)
def test_e8_linear_forward_matches_reference(golden, e8_table, name):
    g = golden("golden_e8_linear.npz")
    W, (fin, fout, m_pad, n_pad) = _e8_rot_weight(g, name, e8_table)
    y = O.linear_forward(g[name + "_x"], W, g[name + "_SU"], g[name + "_SV"], float(g[name + "_Wscale"]),
                         list(g[name + "_blocks_n"]), list(g[name + "_blocks_m"]), fout)
    ref = g[name + "_y"]
    assert np.abs(y - ref).max() <= 2e-5 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("name", ["pow2_1s", "pow2_2s_small"])
def test_e8_dequantize_matches_reference(golden, e8_table, name):
    g = golden("golden_e8_linear.npz")
    W, (fin, fout, m_pad, n_pad) = _e8_rot_weight(g, name, e8_table)
    W = W * np.float32(g[name + "_Wscale"])
    Wt = O.fht(W) * g[name + "_SV"].astype(np.float32)[None, :]
    Wt = O.fht(Wt.T).T * g[name + "_SU"].astype(np.float32)[:, None]
    np.testing.assert_allclose(Wt[:fout, :fin], g[name + "_dequant"], atol=1e-6)


@pytest.mark.parametrize("name", ["k2", "k3", "k4", "k4p2", "k4p4"])
def test_trellis_linear_forward_matches_reference(golden, name):
    g = golden("golden_trellis_linear.npz")
    fin, fout, K, K2 = [int(v) for v in g[name + "_meta"]]
    if K2:
        W = O.trellis_decode_layer_nstage([g[name + "_packed"], g[name + "_packed2"]], [K, K2],
                                          [1.0, float(g[name + "_inv_resid_scale2"])], fout, fin)
    else:
        W = O.trellis_decode_layer(g[name + "_packed"], fout, fin, K).astype(np.float32)
    y = O.linear_forward(g[name + "_x"], W, g[name + "_SU"], g[name + "_SV"], float(g[name + "_Wscale"]))
    ref = g[name + "_y"]
    assert np.abs(y - ref).max() <= 2e-5 * max(1.0, np.abs(ref).max())


def test_moe_forward_matches_dense_loop():
    rng = np.random.default_rng(3)
    T, H, I, E, k = 6, 16, 8, 4, 2
    W13 = rng.standard_normal((E, 2 * I, H)).astype(np.float32)
    W2 = rng.standard_normal((E, H, I)).astype(np.float32)
    x = rng.standard_normal((T, H)).astype(np.float32)
    ids = np.stack([rng.permutation(E)[:k] for _ in range(T)])
    w = rng.random((T, k)).astype(np.float32)
    out = O.moe_forward(x, ids, w, lambda e, xb: xb @ W13[e].T, lambda e, hb: hb @ W2[e].T, I, "silu")
    ref = np.zeros_like(out)
    for t in range(T):
        for j in range(k):
            e = ids[t, j]
            h = W13[e] @ x[t]
            g, u = h[:I], h[I:]
            ref[t] += w[t, j] * (W2[e] @ ((g / (1 + np.exp(-g))) * u))
    np.testing.assert_allclose(out, ref, rtol=1e-5, atol=1e-5)
