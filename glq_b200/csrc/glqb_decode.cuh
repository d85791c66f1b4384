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
  return ((state16 * MUL3 + ADD3) & MASK3) ^ XOR3;
}

// Two hashed states -> half2 (value0, value1); each value = hi half + lo half, added in fp16.
__device__ __forceinline__ uint32_t pair3(uint32_t r0, uint32_t r1) {
  uint32_t lo = __byte_perm(r0, r1, 0x5410);
  uint32_t hi = __byte_perm(r0, r1, 0x7632);
  __half2 v = __hadd2(*reinterpret_cast<__half2*>(&hi), *reinterpret_cast<__half2*>(&lo));
  return *reinterpret_cast<uint32_t*>(&v);
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

// Decode the 8 weights a lane owns in one 16x16 tile into the four registers of an
// m16n8k16 A fragment.  c = this lane's chunk, cn / cn2 = the chunks of lanes +1 / +2 of the same
// tile (cyclic).  Weight j has state = stream bits [K*j, K*j+16) counted from the top of c.
template <int K>
__device__ __forceinline__ void decode_tile(uint32_t c, uint32_t cn, uint32_t cn2, uint32_t (&a)[4]) {
  uint32_t hi, lo;
  if constexpr (K == 4) {
    hi = c; lo = cn;
  } else if constexpr (K == 3) {
    hi = (c << 8) | (cn >> 16); lo = cn << 16;
  } else if constexpr (K == 2) {
    hi = (c << 16) | cn; lo = 0;
  } else {
    hi = (c << 24) | (cn << 16) | (cn2 << 8); lo = 0;
  }
  uint32_t r[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint32_t top = (K * j == 0) ? hi : __funnelshift_l(lo, hi, K * j);
    r[j] = hash3(top >> 16);
  }
#pragma unroll
  for (int p = 0; p < 4; ++p) a[p] = pair3(r[2 * p], r[2 * p + 1]);
}

// Position of weight (lane, j) inside its 16x16 tile.
__device__ __forceinline__ int tile_row(int lane, int j) { return 8 * ((j >> 1) & 1) + (lane >> 2); }
__device__ __forceinline__ int tile_col(int lane, int j) { return 8 * ((j >> 2) & 1) + 2 * (lane & 3) + (j & 1); }

// ------------------------------------------------------------------------------------------
// E8 shell entries: one uint32 per codebook row, nibble i = 2*coord_i + 6
// (reference: glq/codebook.py:102-115).  Values are multiples of 1/2 in [-3, 3], exact in fp16.
// ------------------------------------------------------------------------------------------
// nibbles (i, i+4) -> half2 (coord_i, coord_{i+4}) via the 1024+n mantissa trick:
// (0x6400 | n) is the fp16 number 1024 + n;  (1024 + n) * 0.5 - 515 = n/2 - 3.
__device__ __forceinline__ void e8_entry_to_half2(uint32_t e, uint32_t (&h)[4]) {
  const __half2 half = __floats2half2_rn(0.5f, 0.5f);
  const __half2 bias = __floats2half2_rn(-515.0f, -515.0f);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t v = ((e >> (4 * i)) & 0x000F000Fu) | 0x64006400u;   // (n_i, n_{i+4})
    __half2 r = __hfma2(*reinterpret_cast<__half2*>(&v), half, bias);
    h[i] = *reinterpret_cast<uint32_t*>(&r);
  }
}

__device__ __forceinline__ float e8_coord(uint32_t e, int i) {
  return static_cast<float>((e >> (4 * i)) & 0xFu) * 0.5f - 3.0f;
}

}  // namespace glqb
