"""CPU oracle for the GLQ compressed-weight matmul path.  TEST INFRASTRUCTURE ONLY.

This file restates, in numpy, the reference's algorithm for decoding GLQ's packed
weights and applying a quantised linear layer.  It is the checker the CUDA kernels
are compared against; nothing on the product path may import it (only the test
suite, the smoke check and the CPU-baseline leg of the benchmark do).

Parity status: PINNED.  Every function below is checked bit-for-bit (integer and
fp16 decode) or to fp32 round-off (transforms, layer outputs) against outputs of the
reference itself, stored as fixtures in ``tests/golden/`` by
``tests/golden/make_golden.py`` (which imports the reference package), and against
the known-answer values the reference's own tests hold (shell sizes, FHT values,
block decomposition, permutation inverse).

Reference citations are paths inside the cnygaard/glq project.
"""
from __future__ import annotations

import math

import numpy as np

# --------------------------------------------------------------------------------------
# 3INST arithmetic decode  (glq/trellis.py:122-134 ``decode_3inst``;
# device form glq/csrc/glq_trellis.cu:138-143 ``tr_decode_3inst_half``)
# --------------------------------------------------------------------------------------
MUL_3INST = 89226354
ADD_3INST = 64248484
MASK_3INST = 0x8FFF8FFF
XOR_3INST = 0x3B603B60  # == 996162400


def decode_3inst(state: np.ndarray) -> np.ndarray:
    """16-bit trellis state -> fp16 weight.

    h = state*MUL + ADD (mod 2^32); r = (h & MASK) ^ XOR; the two 16-bit halves of r
    are read as fp16 bit patterns and added IN fp16 (round-to-nearest-even).
    """
    s = np.asarray(state).astype(np.uint64) & np.uint64(0xFFFF)
    h = (s * np.uint64(MUL_3INST) + np.uint64(ADD_3INST)) & np.uint64(0xFFFFFFFF)
    r = ((h & np.uint64(MASK_3INST)) ^ np.uint64(XOR_3INST)).astype(np.uint32)
    hi = (r >> np.uint32(16)).astype(np.uint16).view(np.float16)
    lo = (r & np.uint32(0xFFFF)).astype(np.uint16).view(np.float16)
    return (hi + lo).astype(np.float16)


def table_3inst() -> np.ndarray:
    """All 65,536 decoded values (the reference's ``lut`` buffer, glq/trellis.py:184)."""
    return decode_3inst(np.arange(65536, dtype=np.uint32))


# --------------------------------------------------------------------------------------
# Trellis "kernel" storage layout  (glq/trellis.py:486-523 pack/unpack, :99-101
# _PERMUTE, :580-602 kernel_tile_flip, :629-643 decode_layer)
#
# Restated layout (per stage, K bits per weight, K in 1..4):
#   * the (m, n) matrix is cut into 16x16 tiles; tiles are grouped 2x2 into 32x32
#     groups stored row-major over (row-pair rp, col-pair cp); a group is 128*K bytes;
#   * inside a group bytes are indexed (lane 0..31, ni 0..1, mi 0..1, byte 0..K-1);
#     (mi, ni) picks the tile (row-tile 2rp+mi, col-tile 2cp+ni); the K bytes form one
#     little-endian integer "chunk" of 8K bits;
#   * a tile's bit stream is its 32 chunks (lane order), each MSB first, cyclic;
#   * weight p = 8*lane + j has state = stream bits [p*K, p*K+16) (wrapping);
#   * (lane, j) sits at row 8a+g, col 8c+2t+e with g=lane>>2, t=lane&3,
#     c=(j>>2)&1, a=(j>>1)&1, e=j&1.
# --------------------------------------------------------------------------------------
def _tile_position_maps():
    lane = np.arange(32)[:, None]
    j = np.arange(8)[None, :]
    g, t = lane >> 2, lane & 3
    c, a, e = (j >> 2) & 1, (j >> 1) & 1, j & 1
    row = 8 * a + g
    col = 8 * c + 2 * t + e
    return np.broadcast_to(row, (32, 8)).copy(), np.broadcast_to(col, (32, 8)).copy()


_TILE_ROW, _TILE_COL = _tile_position_maps()


def trellis_states(packed: np.ndarray, m: int, n: int, K: int) -> np.ndarray:
    """packed int16 [(m/16)*(n/16), 16*K] -> uint16 states laid out as the (m, n) matrix."""
    assert m % 32 == 0 and n % 32 == 0, "kernel layout needs whole 32x32 groups"
    assert 1 <= K <= 4
    b = np.ascontiguousarray(packed).view(np.uint8).reshape(-1)
    assert b.size == m * n * K // 8, (b.size, m, n, K)
    RP, CP = m // 32, n // 32
    # (rp, cp, lane, ni, mi, byte)
    g = b.reshape(RP, CP, 32, 2, 2, K).astype(np.uint64)
    chunk = np.zeros((RP, CP, 32, 2, 2), dtype=np.uint64)
    for k in range(K):
        chunk |= g[..., k] << np.uint64(8 * k)           # little-endian
    # per-tile stream as one big integer is awkward in numpy: go through bits
    nb = 8 * K
    shifts = np.arange(nb - 1, -1, -1, dtype=np.uint64)    # MSB first
    bits = ((chunk[..., None] >> shifts) & np.uint64(1)).astype(np.uint8)   # (RP,CP,32,2,2,nb)
    bits = np.moveaxis(bits, 2, 4)                         # (RP,CP,ni,mi,32,nb)
    stream = bits.reshape(RP, CP, 2, 2, 32 * nb)           # 256*K bits per tile
    ext = np.concatenate([stream, stream[..., :16]], axis=-1)
    idx = (np.arange(256) * K)[:, None] + np.arange(16)[None, :]           # (256,16)
    w = (1 << np.arange(15, -1, -1)).astype(np.uint32)
    st = (ext[..., idx].astype(np.uint32) * w).sum(-1).astype(np.uint16)   # (RP,CP,ni,mi,256)
    st = st.reshape(RP, CP, 2, 2, 32, 8)
    out = np.zeros((m, n), dtype=np.uint16)
    rows = _TILE_ROW
    cols = _TILE_COL
    for ni in range(2):
        for mi in range(2):
            # out[32rp + 16mi + row, 32cp + 16ni + col] = st[rp, cp, ni, mi, lane, j]
            view = out.reshape(RP, 32, CP, 32)
            view[:, 16 * mi + rows, :, 16 * ni + cols] = np.transpose(
                st[:, :, ni, mi], (2, 3, 0, 1))
    return out


def trellis_decode_layer(packed: np.ndarray, m: int, n: int, K: int) -> np.ndarray:
    """Oracle for one stage: packed -> fp16 weights (m, n) in the rotated domain
    (glq/trellis.py:629-643 ``decode_layer`` with the 3INST codebook, kernel layout)."""
    return decode_3inst(trellis_states(packed, m, n, K))


def trellis_decode_layer_nstage(packed_list, K_list, cum_inv_rs, m, n) -> np.ndarray:
    """sum_s decode(stage_s) * cum_inv_rs[s], fp32, left to right
    (glq/trellis.py:923-933 ``decode_layer_nstage``; the reference multiplies the float
    tensor by a Python float, i.e. an fp32 multiply, then adds)."""
    out = None
    for packed, K, sc in zip(packed_list, K_list, cum_inv_rs):
        d = trellis_decode_layer(packed, m, n, K).astype(np.float32) * np.float32(sc)
        out = d if out is None else (out + d).astype(np.float32)
    return out


def trellis_pack_states(states: np.ndarray, K: int) -> np.ndarray:
    """Inverse of :func:`trellis_states` for VALID tail-biting state matrices (used only
    to build test inputs): states (m, n) uint16 -> packed int16 [(m/16)(n/16), 16K]."""
    m, n = states.shape
    RP, CP = m // 32, n // 32
    view = states.reshape(RP, 32, CP, 32)
    packed = np.zeros((RP, CP, 32, 2, 2, K), dtype=np.uint8)
    for ni in range(2):
        for mi in range(2):
            st = np.transpose(view[:, 16 * mi + _TILE_ROW, :, 16 * ni + _TILE_COL],
                              (2, 3, 0, 1)).reshape(RP, CP, 256).astype(np.uint32)
            # new bits of weight p are the low K bits of state p+? : stream bits
            # [p*K, p*K+16) = state p  => stream bits [p*K, p*K+K) = top K bits of state p
            top = (st >> np.uint32(16 - K)) & np.uint32((1 << K) - 1)       # (RP,CP,256)
            sh = np.arange(K - 1, -1, -1, dtype=np.uint32)
            bits = ((top[..., None] >> sh) & 1).astype(np.uint8).reshape(RP, CP, 32, 8 * K)
            w = (np.uint64(1) << np.arange(8 * K - 1, -1, -1, dtype=np.uint64))
            chunk = (bits.astype(np.uint64) * w).sum(-1)                   # (RP,CP,32)
            for k in range(K):
                packed[:, :, :, ni, mi, k] = ((chunk >> np.uint64(8 * k)) & np.uint64(0xFF)).astype(np.uint8)
    return packed.reshape(-1).view(np.int16).reshape((m // 16) * (n // 16), 16 * K)


# --------------------------------------------------------------------------------------
# E8 shell codebook decode  (glq/codebook.py:280-282 ``decode``; packed nibble form
# glq/codebook.py:102-115 ``_pack_codebook``; N-stage sum glq/quantized_linear.py:1177-1194)
# --------------------------------------------------------------------------------------
E8_SHELL_SIZES = [1, 240, 2160, 6720, 17520, 30240, 60480]   # glq/codebook.py:169-171


def e8_unpack_table(packed_u32: np.ndarray) -> np.ndarray:
    """uint32 nibble-packed table (code = 2*coord + 6 in nibble i) -> fp32 (K, 8)."""
    p = np.asarray(packed_u32).astype(np.uint32)
    sh = (4 * np.arange(8)).astype(np.uint32)
    nib = (p[:, None] >> sh) & np.uint32(0xF)
    return nib.astype(np.float32) * np.float32(0.5) - np.float32(3.0)


def e8_pack_table(table: np.ndarray) -> np.ndarray:
    codes = np.rint(np.asarray(table, dtype=np.float64) * 2.0).astype(np.int64) + 6
    assert codes.min() >= 0 and codes.max() <= 12
    out = np.zeros(table.shape[0], dtype=np.uint32)
    for i in range(8):
        out |= (codes[:, i].astype(np.uint32) << np.uint32(4 * i))
    return out


def e8_decode(qidxs: np.ndarray, table: np.ndarray) -> np.ndarray:
    """int16 (m, n/8) indices (bit pattern read as uint16) -> fp32 (m, n)."""
    q = np.ascontiguousarray(qidxs).view(np.uint16).astype(np.int64)
    m, nb = q.shape
    return table[q.reshape(-1) % table.shape[0]].reshape(m, nb * 8).astype(np.float32)


def e8_decode_nstage(qidxs_list, tables, inv_rs) -> np.ndarray:
    """W = cb[q1]; W = W + cb_s[q_s] * inv_rs[s-1] for s = 2.. (fp32 multiply THEN fp32
    add, no fused multiply-add; stages in order) — glq/quantized_linear.py:1177-1194."""
    W = e8_decode(qidxs_list[0], tables[0])
    for q, tb, s in zip(qidxs_list[1:], tables[1:], inv_rs):
        Ws = (e8_decode(q, tb) * np.float32(s)).astype(np.float32)
        W = (W + Ws).astype(np.float32)
    return W


# --------------------------------------------------------------------------------------
# Walsh-Hadamard / block-diagonal RHT  (glq/hadamard.py:10-28 ``_pytorch_fht``,
# :133-146 ``_block_decompose``, :166-178 ``block_diagonal_fht``)
# --------------------------------------------------------------------------------------
def block_decompose(n: int) -> list[int]:
    out = []
    while n > 0:
        p = 1 << (n.bit_length() - 1)
        out.append(p)
        n -= p
    return out


def fht(x: np.ndarray) -> np.ndarray:
    """Orthonormal Walsh-Hadamard transform along the last axis (power-of-two length).
    Stages in ascending distance; lower index gets a+b, upper a-b; one division by sqrt(n)."""
    x = np.array(x, dtype=np.float32, copy=True)
    n = x.shape[-1]
    assert n > 0 and n & (n - 1) == 0
    h = 1
    while h < n:
        v = x.reshape(*x.shape[:-1], n // (2 * h), 2, h)
        a = v[..., 0, :].copy()
        b = v[..., 1, :].copy()
        v[..., 0, :] = a + b
        v[..., 1, :] = a - b
        x = v.reshape(*x.shape)
        h *= 2
    return (x / np.float32(math.sqrt(n))).astype(np.float32)


def block_diag_fht(x: np.ndarray, blocks) -> np.ndarray:
    x = np.array(x, dtype=np.float32, copy=True)
    off = 0
    for bs in blocks:
        x[..., off:off + bs] = fht(x[..., off:off + bs])
        off += bs
    return x


# --------------------------------------------------------------------------------------
# Quantised linear layer: y = [SU * H_m( Wscale * W~ . H_n(SV * pad(x)) )][:out]
# (glq/quantized_linear.py:1149-1154, 1176-1195, 1225-1231 E8 CPU path;
#  :986-1010 trellis CPU path)
# --------------------------------------------------------------------------------------
def linear_forward(x, W_rot, SU, SV, wscale, blocks_n=None, blocks_m=None,
                   out_features=None, row_scale=None):
    """fp32 reference of one GLQ linear.  x (B, in), W_rot (m_pad, n_pad) rotated-domain
    weights (unscaled), SU (m_pad,), SV (n_pad,).  ``row_scale`` (m_pad,) is the
    per-row-scale superset used only by the synthetic benchmark config; the stored
    reference layer has the single scalar ``wscale``."""
    x = np.asarray(x, dtype=np.float32)
    m_pad, n_pad = W_rot.shape
    B, in_f = x.shape
    blocks_n = blocks_n or block_decompose(n_pad)
    blocks_m = blocks_m or block_decompose(m_pad)
    xp = np.zeros((B, n_pad), dtype=np.float32)
    xp[:, :in_f] = x
    xr = block_diag_fht(xp * np.asarray(SV, dtype=np.float32)[None, :], blocks_n)
    yr = (xr @ np.asarray(W_rot, dtype=np.float32).T) * np.float32(wscale)
    if row_scale is not None:
        yr = yr * np.asarray(row_scale, dtype=np.float32)[None, :]
    y = block_diag_fht(yr, blocks_m) * np.asarray(SU, dtype=np.float32)[None, :]
    out_features = out_features or m_pad
    return y[:, :out_features].astype(np.float32)


# --------------------------------------------------------------------------------------
# MoE: out[t] = sum_k w[t,k] * W2_e( act(W13_e x_t) ), e = ids[t,k]
# (glq_vllm/fused_moe_method.py:393-440 eager loop, :31-62 activations)
# --------------------------------------------------------------------------------------
def _act(name):
    if name == "silu":
        return lambda g: g / (1.0 + np.exp(-g))
    if name == "gelu_tanh":
        return lambda g: 0.5 * g * (1.0 + np.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
    if name in ("relu2", "relu2_no_mul"):
        return lambda g: np.square(np.maximum(g, 0.0))
    if name == "silu_no_mul":
        return lambda g: g / (1.0 + np.exp(-g))
    if name == "gelu_no_mul":                      # F.gelu with the exact (erf) form
        from math import erf
        verf = np.vectorize(erf, otypes=[np.float64])
        return lambda g: (0.5 * g * (1.0 + verf(g.astype(np.float64) * 0.7071067811865476))).astype(np.float32)
    raise ValueError(name)


# integer codes of the fused ops (glq_vllm/fused_moe_method.py:671-677): 0-2 gated, 3-5 without the gate
ACT_CODES = {0: "silu", 1: "gelu_tanh", 2: "relu2", 3: "silu_no_mul", 4: "gelu_no_mul", 5: "relu2_no_mul"}


def moe_forward(x, topk_ids, topk_w, expert_fn13, expert_fn2, inter, activation="gelu_tanh"):
    """expert_fn13(e, xb) -> (b, 2*inter) [gate; up], expert_fn2(e, hb) -> (b, hidden)."""
    x = np.asarray(x, dtype=np.float32)
    T, H = x.shape
    out = np.zeros((T, H), dtype=np.float32)
    act = _act(activation)
    for e in np.unique(topk_ids):
        tok, slot = np.nonzero(topk_ids == e)
        if tok.size == 0:
            continue
        h13 = expert_fn13(int(e), x[tok]).astype(np.float32)
        if activation.endswith("_no_mul"):         # w13 has `inter` rows: no up projection
            h = act(h13[:, :inter]).astype(np.float32)
        else:
            h = (act(h13[:, :inter]) * h13[:, inter:2 * inter]).astype(np.float32)
        y = expert_fn2(int(e), h)
        np.add.at(out, tok, y * np.asarray(topk_w, dtype=np.float32)[tok, slot][:, None])
    return out
