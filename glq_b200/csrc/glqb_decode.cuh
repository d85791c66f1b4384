// Device-side decoders shared by the matvec, GEMM and dump kernels, so that the weights the
// compute kernels reconstruct are, by construction, the ones the dump kernels write out.
#pragma once
#include "glqb_internal.h"

namespace glqb {

// ------------------------------------------------------------------------------------------
// 3INST arithmetic decode (reference: glq/trellis.py:122-134, glq/csrc/glq_trellis.cu:138-143)
// state (16 bit) -> h = state*MUL + ADD (mod 2^32) -> r = (h & MASK) ^ XOR -> fp16(r.hi) + fp16(r.lo)
// ------------------------------------------------------------------------------------------
constexpr uint32_t MUL3 = 89226354u;
constexpr uint32_t ADD3 = 64248484u;
constexpr uint32_t MASK3 = 0x8FFF8FFFu;
constexpr uint32_t XOR3 = 0x3B603B60u;

__device__ __forceinline__ uint32_t hash3(uint32_t state16) {
  const uint32_t h = state16 * MUL3 + ADD3;
  uint32_t r;
  // (h & MASK) ^ XOR as ONE three-input logic op (truth table 0x6A), both constants in registers
  asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(r) : "r"(h), "r"(MASK3), "r"(XOR3));
  return r;
}

// One hashed state -> half2 (v, v) with v = fp16(hi half) + fp16(lo half), the addition done in fp16
// (round to nearest even) exactly as the reference does.  Both halves of the result carry v: the MMA
// then takes the register as an A-fragment entry whose two k slots meet (x, 0) in the B fragment, so
// no instruction is spent on packing two different weights into one register.
__device__ __forceinline__ uint32_t sum_dup3(uint32_t r) {
  const __half2 v = *reinterpret_cast<const __half2*>(&r);
  const __half2 s = __hadd2(__low2half2(v), __high2half2(v));
  return *reinterpret_cast<const uint32_t*>(&s);
}

// A lane's share of one 32x32 group is 4*K bytes = K 32-bit words, holding four chunks of 8K bits
// ordered (ni, mi) = (0,0),(0,1),(1,0),(1,1); chunk q sits at bits [8K*q, 8K*q+8K) of the
// little-endian integer formed by the words.
template <int K>
struct Words {
  uint32_t w[K];
};

template <int K>
__device__ __forceinline__ uint32_t chunk_of(const Words<K>& v, int q) {
  if constexpr (K == 4) {
    return v.w[q];
  } else if constexpr (K == 2) {
    return (q & 1) ? (v.w[q >> 1] >> 16) : (v.w[q >> 1] & 0xFFFFu);
  } else if constexpr (K == 1) {
    return (v.w[0] >> (8 * q)) & 0xFFu;
  } else {  // K == 3: 24-bit chunks over three words
    if (q == 0) return v.w[0] & 0xFFFFFFu;
    if (q == 1) return (v.w[0] >> 24) | ((v.w[1] & 0xFFFFu) << 8);
    if (q == 2) return (v.w[1] >> 16) | ((v.w[2] & 0xFFu) << 16);
    return v.w[2] >> 8;
  }
}

// The 8 states a lane owns in one 16x16 tile.  c = this lane's chunk, cn / cn2 = the chunks of
// lanes +1 / +2 of the same tile (cyclic).  Weight j has state = stream bits [K*j, K*j+16) counted
// from the top of c.
template <int K>
__device__ __forceinline__ void tile_states(uint32_t c, uint32_t cn, uint32_t cn2, uint32_t (&s)[8]) {
  if constexpr (K == 4) {
    // 64-bit window {c, cn}; states start every 4 bits.  Even states are byte aligned in the window,
    // odd states are byte aligned in the window shifted left by 4: every state is one byte permute
    // (zero-filled upper half) of c, c<<4, w2 = window bits [16,48) or w2<<4.
    const uint32_t w2 = __byte_perm(cn, c, 0x5432);
    const uint32_t t1 = c << 4;
    const uint32_t t2 = w2 << 4;
    s[0] = __byte_perm(c, 0u, 0x4432);
    s[1] = __byte_perm(t1, 0u, 0x4432);
    s[2] = __byte_perm(c, 0u, 0x4421);
    s[3] = __byte_perm(t1, 0u, 0x4421);
    s[4] = __byte_perm(c, 0u, 0x4410);
    s[5] = __byte_perm(t2, 0u, 0x4432);
    s[6] = __byte_perm(w2, 0u, 0x4421);
    s[7] = __byte_perm(t2, 0u, 0x4421);
  } else {
    uint32_t hi, lo;
    if constexpr (K == 3) {
      hi = (c << 8) | (cn >> 16); lo = cn << 16;
    } else if constexpr (K == 2) {
      hi = (c << 16) | cn; lo = 0;
    } else {
      hi = (c << 24) | (cn << 16) | (cn2 << 8); lo = 0;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t top = (K * j == 0) ? hi : ((K * j + 16 <= 32) ? (hi << (K * j)) : __funnelshift_l(lo, hi, K * j));
      s[j] = top >> 16;
    }
  }
}

// Decode a lane's 8 weights of a tile: a[j] = half2 (w_j, w_j).
// LUT > 0: the first LUT of a lane's 8 states are looked up in a table of all 65,536 fp16 values of the code that
// the CTA keeps in shared memory (`lut_base`: its shared-window address) instead of being computed.  The
// arithmetic decode saturates the integer/logic pipes while the load/store pipe idles; moving a quarter of the
// states over balances them (measured on B200, 4-bit rate, fraction of the measured HBM rate: 0 of 8 states
// 0.356, 1: 0.379, 2: 0.385, 3: 0.349, 4: 0.286 — beyond two the random bank conflicts of the loads dominate).
// Same values by construction: the table is filled with the arithmetic decode itself.
template <int K, int LUT = 0>
__device__ __forceinline__ void decode_tile(uint32_t c, uint32_t cn, uint32_t cn2, uint32_t (&a)[8], uint32_t lut_base = 0u) {
  uint32_t s[8];
  tile_states<K>(c, cn, cn2, s);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    if (j < LUT) {
      // the table holds the fp16 value of every state; the upper half of the A entry meets a zero in B
      unsigned short v;
      asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(lut_base + (s[j] << 1)));
      a[j] = v;
    } else {
      a[j] = sum_dup3(hash3(s[j]));
    }
  }
}

// Position of weight (lane, j) inside its 16x16 tile.
__device__ __forceinline__ int tile_row(int lane, int j) { return 8 * ((j >> 1) & 1) + (lane >> 2); }
__device__ __forceinline__ int tile_col(int lane, int j) { return 8 * ((j >> 2) & 1) + 2 * (lane & 3) + (j & 1); }

// ------------------------------------------------------------------------------------------
// E8 shell entries: one uint32 per codebook row, nibble i = 2*coord_i + 6
// (reference: glq/codebook.py:102-115).  Values are multiples of 1/2 in [-3, 3], exact in fp16.
// ------------------------------------------------------------------------------------------
// nibbles (i, i+4) -> half2 (coord_i, coord_{i+4}) via the mantissa trick: (0x6400 | n) is the fp16
// number 1024 + n, so (1024 + n) * 0.5 - 515 = n/2 - 3; a nibble sitting four bits higher gives
// 1024 + 16 n, and (1024 + 16 n) / 32 - 35 = n/2 - 3 as well (all steps exact in fp16).  Odd nibbles
// therefore need no shift: one shift (by 8) serves nibbles 2 and 3.
__device__ __forceinline__ void e8_entry_to_half2(uint32_t e, uint32_t (&h)[4]) {
  const __half2 half = __floats2half2_rn(0.5f, 0.5f);
  const __half2 bias = __floats2half2_rn(-515.0f, -515.0f);
  const __half2 half16 = __floats2half2_rn(0.03125f, 0.03125f);
  const __half2 bias16 = __floats2half2_rn(-35.0f, -35.0f);
  const uint32_t e8 = e >> 8;
  uint32_t v0 = (e & 0x000F000Fu) | 0x64006400u;    // (n0, n4)
  uint32_t v1 = (e & 0x00F000F0u) | 0x64006400u;    // 16 * (n1, n5)
  uint32_t v2 = (e8 & 0x000F000Fu) | 0x64006400u;   // (n2, n6)
  uint32_t v3 = (e8 & 0x00F000F0u) | 0x64006400u;   // 16 * (n3, n7)
  __half2 r0 = __hfma2(*reinterpret_cast<__half2*>(&v0), half, bias);
  __half2 r1 = __hfma2(*reinterpret_cast<__half2*>(&v1), half16, bias16);
  __half2 r2 = __hfma2(*reinterpret_cast<__half2*>(&v2), half, bias);
  __half2 r3 = __hfma2(*reinterpret_cast<__half2*>(&v3), half16, bias16);
  h[0] = *reinterpret_cast<uint32_t*>(&r0);
  h[1] = *reinterpret_cast<uint32_t*>(&r1);
  h[2] = *reinterpret_cast<uint32_t*>(&r2);
  h[3] = *reinterpret_cast<uint32_t*>(&r3);
}

__device__ __forceinline__ float e8_coord(uint32_t e, int i) {
  return static_cast<float>((e >> (4 * i)) & 0xFu) * 0.5f - 3.0f;
}

}  // namespace glqb
