// Kernels of the decode (small-batch) path: input transform, streaming decode + mma, output transform,
// and the dump kernels used by the bit-exact gate.
#pragma once
#include "glqb_internal.h"
#include "glqb_decode.cuh"
#include "glqb_fht.cuh"
#include "glqb_comm.cuh"

namespace glqb {

#ifndef GLQB_LUT_THREADS
#define GLQB_LUT_THREADS 768
#endif
constexpr int MV_THREADS = 256;               // 8 warps per CTA in the streaming kernels
constexpr int MV_WARPS = MV_THREADS / 32;

// ---------------------------------------------------------------------------------------------
// small helpers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float load_act(const void* base, long long idx, int dtype) {
  if (dtype == GLQB_DT_F16) return __half2float(reinterpret_cast<const __half*>(base)[idx]);
  if (dtype == GLQB_DT_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[idx]);
  return reinterpret_cast<const float*>(base)[idx];
}

__device__ __forceinline__ void store_act(void* base, long long idx, int dtype, float v) {
  if (dtype == GLQB_DT_F16) reinterpret_cast<__half*>(base)[idx] = __float2half_rn(v);
  else if (dtype == GLQB_DT_BF16) reinterpret_cast<__nv_bfloat16*>(base)[idx] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(base)[idx] = v;
}

// four consecutive activations; idx must be a multiple of 4 and the row 8/16-byte aligned (the callers
// check) — one 8- or 16-byte access instead of four
__device__ __forceinline__ void load_act4(const void* base, long long idx, int dtype, float (&v)[4]) {
  if (dtype == GLQB_DT_F32) {
    const float4 t = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + idx);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  } else {
    const uint2 t = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(base) + idx);
    if (dtype == GLQB_DT_F16) {
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t.x));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
      v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    } else {
      v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xFFFF0000u);
      v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xFFFF0000u);
    }
  }
}
__device__ __forceinline__ void store_act4(void* base, long long idx, int dtype, const float (&v)[4]) {
  if (dtype == GLQB_DT_F32) {
    *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + idx) = make_float4(v[0], v[1], v[2], v[3]);
  } else if (dtype == GLQB_DT_F16) {
    const __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(base) + idx) =
        make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
  } else {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(base) + idx) =
        make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
  }
}
__device__ __forceinline__ bool act_rows_aligned4(const void* base, long long off, long long stride, int dtype) {
  const int es = dtype == GLQB_DT_F32 ? 4 : 2;
  return ((off | stride) & 3) == 0 && (reinterpret_cast<uintptr_t>(base) & (4 * es - 1)) == 0;
}

// value after a round trip through the activation dtype (what a separate kernel would have stored)
__device__ __forceinline__ float round_act(float v, int dtype) {
  if (dtype == GLQB_DT_F16) return __half2float(__float2half_rn(v));
  if (dtype == GLQB_DT_BF16) return __bfloat162float(__float2bfloat16_rn(v));
  return v;
}
// gated / plain activations of the MoE ops and of the fused decode input (GLQB_ACT_*)
__device__ __forceinline__ float act_fn(float g, int act) {
  if (act == GLQB_ACT_SILU) return g / (1.0f + __expf(-g));
  if (act == GLQB_ACT_GELU_TANH) {
    const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.0f + tanhf(u));
  }
  const float r = fmaxf(g, 0.f);
  return r * r;
}

// streaming 128/64/32-bit loads of weight codes: read once, keep out of L1
__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint2 ld_stream_v2(const void* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ld_stream_u32(const void* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Trellis activations are stored per 32-column group as 64 halfs: column c = 16ni + 8h + 2t + e sits at
// half index t*16 + ni*8 + e*4 + h*2 and is followed by a zero, i.e. every B-fragment register of
// the MMA is (x, 0).  Lane t fetches its 32 bytes of a group with two 16-byte loads (one per ni).
constexpr int XR_TRELLIS_EXPAND = 2;   // halfs stored per activation
__device__ __forceinline__ int xr_pos_trellis(int c) {
  int ni = c >> 4, h = (c >> 3) & 1, t = (c >> 1) & 3, e = c & 1;
  return t * 16 + ni * 8 + e * 4 + h * 2;
}
// position of column i (0..7) of an E8 block: (x0,x4,x1,x5,x2,x6,x3,x7)
__device__ __forceinline__ int xr_pos_e8(int i) { return (i & 3) * 2 + (i >> 2); }
// E8 activations for the streaming kernel.  One token: 8-column blocks in order.  Several tokens: the
// blocks of 8 consecutive tokens are interleaved (token group, block, token in group, 8 halfs), so that
// the 8 tokens a warp multiplies against one block sit in one 128-byte line instead of eight.
__device__ __forceinline__ long long xr_index_e8(long long token, int col, int n, int batch) {
  const int j = xr_pos_e8(col & 7);
  if (batch == 1) return (col & ~7) + j;
  return ((((token >> 3) * (n >> 3) + (col >> 3)) << 3) + (token & 7)) * 8 + j;
}

// ---------------------------------------------------------------------------------------------
// Input transform:  xr = fp16( H_blocks( SV * pad(x) ) / sqrt(bs) ), written in the layout the
// decode kernel of the layer's format reads (reference: glq_input_rht_multiblock_kernel,
// glq/csrc/glq_cuda.cu:2092; rounding to fp16 as glq/csrc/glq_cuda.cu:2625).
// One CTA per (layer, Hadamard block, tile of tokens); the transform itself is fht_tile (first pass
// fused with the global loads, last pass with the stores).
// PLAIN_F32: write fp32 in natural order instead (the unfused input_rht op).
// ---------------------------------------------------------------------------------------------
#ifndef GLQB_RHT_THREADS
#define GLQB_RHT_THREADS 256
#endif
#ifndef GLQB_RHT_MINB
#define GLQB_RHT_MINB 4
#endif
constexpr int RHT_THREADS = GLQB_RHT_THREADS;
// longest array the transform kernels hand to the shuffle-based transform (their 64-register budget holds 8
// values per thread plus what travels with them); longer arrays keep the tiled passes
constexpr int RHT_FAST_MAX_LOG = 11;
// The low-latency forms (shuffle transform per token, split blocks) serve launches of a few items, where the
// time of one item is the time of the launch; launches of many items keep the tiled passes, which move more
// values per clock (measured: 252 layers, one token: 33 us for both transforms tiled, 77 us in the low-latency form).
constexpr int RHT_LATENCY_MAX_ITEMS = 128;
constexpr int RHT_SPLIT_LOG = 10;                // run length of the split form (RhtItem::sub): 1024
constexpr int RHT_SPLIT_MIN_LOG = 12;            // blocks of at least 4096 values are split in decode-sized plans

constexpr int FUSED_MAX_TOKENS_C = 8;     // tokens served by the single-launch decode form and its fused steps

// Input value of column `col` of token row starting at element `xt0`, before the sign vector: x itself, or
// act(gate) * up for a [gate | up] row (both factors and the product rounded to the activation dtype, as
// separate kernels would store them).
__device__ __forceinline__ float input_value(const DevLinear& L, const uint8_t* x_base, long long xt0, int col) {
  float v = load_act(x_base, xt0 + col, L.x_dtype);
  if (L.in_gated_act)
    v = round_act(round_act(act_fn(v, L.in_gated_act - 1), L.x_dtype) * load_act(x_base, xt0 + L.in_f + col, L.x_dtype), L.x_dtype);
  return v;
}
// 1 / rms of a token's input values (fused RMSNorm), by all threads of the CTA; `red` holds >= 32 floats
__device__ __forceinline__ float token_rstd(const DevLinear& L, const uint8_t* x_base, long long xt0, float* red) {
  float ss = 0.f;
  for (int i = threadIdx.x; i < L.in_f; i += blockDim.x) { const float v = input_value(L, x_base, xt0, i); ss += v * v; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
  return rsqrtf(tot / (float)L.in_f + L.in_norm_eps);
}

// 32 consecutive activations of one token, times SV, zero past in_features
__device__ __forceinline__ void rht_load_x32(const DevLinear& L, const uint8_t* x_base, long long token, int col0,
                                             bool vec_ok, float (&v)[32]) {
  const long long base = L.x_off + token * L.x_stride;
  const bool rotated = L.x_is_rotated != 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int col = col0 + 4 * j;
    float t[4] = {0.f, 0.f, 0.f, 0.f};
    if (vec_ok && col + 3 < L.in_f) {
      load_act4(x_base, base + col, L.x_dtype, t);
      if (!rotated) {
        const uint2 s4 = *reinterpret_cast<const uint2*>(L.sv + col);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&s4.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&s4.y));
        t[0] *= a.x; t[1] *= a.y; t[2] *= b.x; t[3] *= b.y;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (col + k < L.in_f) {
          t[k] = load_act(x_base, base + col + k, L.x_dtype);
          if (!rotated) t[k] *= __half2float(L.sv[col + k]);
        }
    }
    v[4 * j] = t[0]; v[4 * j + 1] = t[1]; v[4 * j + 2] = t[2]; v[4 * j + 3] = t[3];
  }
}

template <bool PLAIN_F32>
__device__ __forceinline__ void rht_in_body(const DevLinear& L, const RhtItem it, const uint8_t* __restrict__ x_base,
                                            uint8_t* __restrict__ ws, float* fbuf) {
  const int off = L.bn_off[it.block];
  const int logbs = L.bn_log[it.block];
  const int bs = 1 << logbs;
  const bool trellis = (L.format == GLQB_FMT_TRELLIS_3INST);
  const bool vec_ok = (off & 3) == 0 && act_rows_aligned4(x_base, L.x_off, L.x_stride, L.x_dtype);
  const float rs = L.x_is_rotated ? 1.0f : rsqrtf((float)bs);
  auto store1 = [&](int row, int i, float val) {
    const int col = off + i;
    const long long token = it.tok0 + row;
    const float v = val * rs;
    if constexpr (PLAIN_F32) {
      reinterpret_cast<float*>(ws + L.xr_off)[token * L.n + col] = v;
    } else if (trellis) {
      const int pos = (col & ~31) * XR_TRELLIS_EXPAND + xr_pos_trellis(col & 31);   // half index, even
      (reinterpret_cast<__half2*>(ws + L.xr_off) + token * L.n)[pos >> 1] =
          __halves2half2(__float2half_rn(v), __float2half_rn(0.f));
    } else {
      reinterpret_cast<__half*>(ws + L.xr_off)[xr_index_e8(token, col, L.n, L.batch)] = __float2half_rn(v);
    }
  };
  const bool fusions = L.in_gated_act != 0 || L.in_norm_w != nullptr;
  auto load1 = [&](int row, int i) -> float {
    const int col = off + i;
    if (col >= L.in_f) return 0.f;
    const long long xt0 = L.x_off + (long long)(it.tok0 + row) * L.x_stride;
    float v = fusions ? input_value(L, x_base, xt0, col) : load_act(x_base, xt0 + col, L.x_dtype);
    if (L.in_norm_w) v *= load_act(L.in_norm_w, col, L.in_norm_dtype);
    if (!L.x_is_rotated) v *= __half2float(L.sv[col]);
    return v;
  };
  if (L.x_is_rotated) {            // already transformed by the caller: convert and lay out only
    const int total = it.ntok << logbs;
    for (int o = threadIdx.x; o < total; o += blockDim.x) store1(o >> logbs, o & (bs - 1), load1(o >> logbs, o & (bs - 1)));
    return;
  }
  if (it.sub >= 0) {
    // split form: this CTA produces outputs [sub * 1024, sub * 1024 + 1024) of the block (see RhtItem::sub)
    const int S = bs >> RHT_SPLIT_LOG, k = it.sub;
    for (int row = 0; row < it.ntok; ++row) {
      const long long xt0 = L.x_off + (long long)(it.tok0 + row) * L.x_stride;
      float rstd = 1.f;
      if (L.in_norm_w) rstd = token_rstd(L, x_base, xt0, fbuf);
      __syncthreads();
      auto ld1 = [&](int i) -> float {
        float a = 0.f;
        for (int kk = 0; kk < S; ++kk) {
          const float v = load1(row, (kk << RHT_SPLIT_LOG) + i);
          a += (__popc(k & kk) & 1) ? -v : v;
        }
        return a;
      };
      auto ld4 = [&](int i0, float (&q)[4]) {
        q[0] = q[1] = q[2] = q[3] = 0.f;
        for (int kk = 0; kk < S; ++kk) {
          float t[4];
          const int i = (kk << RHT_SPLIT_LOG) + i0;
          if (vec_ok && !fusions && off + i + 3 < L.in_f) {
            load_act4(x_base, xt0 + off + i, L.x_dtype, t);
            const uint2 s4 = *reinterpret_cast<const uint2*>(L.sv + off + i);
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&s4.x));
            const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&s4.y));
            t[0] *= a.x; t[1] *= a.y; t[2] *= c.x; t[3] *= c.y;
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) t[j] = load1(row, i + j);
          }
          const float sg = (__popc(k & kk) & 1) ? -1.f : 1.f;
          q[0] += sg * t[0]; q[1] += sg * t[1]; q[2] += sg * t[2]; q[3] += sg * t[3];
        }
      };
      auto none = [](int) -> float { return 0.f; };
      auto st = [&](int i, float val, float) { store1(row, (k << RHT_SPLIT_LOG) + i, val * rstd); };
      fht_fast<RHT_SPLIT_LOG>(fbuf, RHT_SPLIT_LOG, ld1, ld4, none, st);
      __syncthreads();
    }
    return;
  }
  if (blockDim.x == 256 && L.batch <= FUSED_MAX_TOKENS_C && gridDim.x <= RHT_LATENCY_MAX_ITEMS && logbs >= 5 && logbs <= RHT_FAST_MAX_LOG) {
    // Decode-sized tile (a few tokens): latency matters, not throughput.  Every token's block is transformed by
    // all 256 threads with the shuffle-based transform: one round of loads, one shared-memory exchange.
    const bool plain_vec = vec_ok && !fusions;
    for (int row = 0; row < it.ntok; ++row) {
      const long long xt0 = L.x_off + (long long)(it.tok0 + row) * L.x_stride;
      float rstd = 1.f;
      if (L.in_norm_w) rstd = token_rstd(L, x_base, xt0, fbuf);
      __syncthreads();
      auto ld1 = [&](int i) -> float { return load1(row, i); };
      auto ld4 = [&](int i0, float (&q)[4]) {
        if (plain_vec && off + i0 + 3 < L.in_f) {
          load_act4(x_base, xt0 + off + i0, L.x_dtype, q);
          const uint2 s4 = *reinterpret_cast<const uint2*>(L.sv + off + i0);
          const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&s4.x));
          const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&s4.y));
          q[0] *= a.x; q[1] *= a.y; q[2] *= c.x; q[3] *= c.y;
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) q[k] = load1(row, i0 + k);
        }
      };
      auto none = [](int) -> float { return 0.f; };
      auto st = [&](int i, float val, float) { store1(row, i, val * rstd); };
      fht_fast<RHT_FAST_MAX_LOG>(fbuf, logbs, ld1, ld4, none, st);
      __syncthreads();
    }
    return;
  }
  if (fusions) {
    // fused RMSNorm / gated activation in front of the transform (decode: one token per CTA and block):
    // 1 / rms of the token is folded into the stored values
    float rstd[FUSED_MAX_TOKENS_C];                 // per token of the tile (at most 8 tokens take this path)
#pragma unroll
    for (int r = 0; r < FUSED_MAX_TOKENS_C; ++r) {
      rstd[r] = 1.f;
      if (L.in_norm_w && r < it.ntok) rstd[r] = token_rstd(L, x_base, L.x_off + (long long)(it.tok0 + r) * L.x_stride, fbuf);
    }
    __syncthreads();
    auto store_n = [&](int row, int i, float val) {
      float sc = 1.f;
#pragma unroll
      for (int r = 0; r < FUSED_MAX_TOKENS_C; ++r) if (r == row) sc = rstd[r];
      store1(row, i, val * sc);
    };
    auto load32f = [&](int row, int i0, float (&v)[32]) {
#pragma unroll
      for (int k = 0; k < 32; ++k) v[k] = load1(row, i0 + k);
    };
    fht_tile(fbuf, logbs, it.ntok, load32f, load1, store_n);
    return;
  }
  auto load32 = [&](int row, int i0, float (&v)[32]) { rht_load_x32(L, x_base, it.tok0 + row, off + i0, vec_ok, v); };
  fht_tile(fbuf, logbs, it.ntok, load32, load1, store1);
}

template <bool PLAIN_F32>
__global__ void __launch_bounds__(RHT_THREADS, GLQB_RHT_MINB) rht_in_kernel(const DevLinear* __restrict__ layers,
                                                             const RhtItem* __restrict__ items,
                                                             const uint8_t* __restrict__ x_base,
                                                             uint8_t* __restrict__ ws) {
  extern __shared__ float fbuf[];
  // a successor launched with programmatic stream serialization (the single-launch decode kernel) may start
  // its prologue now; it waits for this kernel's completion before it reads the activations
  asm volatile("griddepcontrol.launch_dependents;");
  const RhtItem it = items[blockIdx.x];
  rht_in_body<PLAIN_F32>(layers[it.layer], it, x_base, ws, fbuf);
}

// One layer described entirely in kernel-parameter space (no device table, nothing to allocate or copy):
// the unfused input_rht / output_rht ops.  CTA b of Hadamard block k handles the token tile
// b - first_cta[k]; tile_tokens[k] tokens per tile.
struct RhtSingle {
  int first_cta[GLQB_MAX_BLOCKS + 1];
  int tile_tokens[GLQB_MAX_BLOCKS];
  int n_blocks;
};
__device__ __forceinline__ RhtItem rht_single_item(const RhtSingle& S, int batch) {
  int k = 0;
  while (k + 1 < S.n_blocks && (int)blockIdx.x >= S.first_cta[k + 1]) ++k;
  const int tok0 = ((int)blockIdx.x - S.first_cta[k]) * S.tile_tokens[k];
  return RhtItem{0, k, tok0, min(S.tile_tokens[k], batch - tok0), -1};
}
static __global__ void __launch_bounds__(RHT_THREADS, GLQB_RHT_MINB) rht_in_single_kernel(const __grid_constant__ DevLinear L,
                                                                    const __grid_constant__ RhtSingle S,
                                                                    const uint8_t* __restrict__ x_base,
                                                                    uint8_t* __restrict__ out) {
  extern __shared__ float fbuf[];
  rht_in_body<true>(L, rht_single_item(S, L.batch), x_base, out, fbuf);
}

// ---------------------------------------------------------------------------------------------
// Output transform: sums the partial sums of every strip in fixed (ascending slot) order, applies
// wscale (and the optional per-row scale), the block Hadamard, 1/sqrt(bs) and SU, and writes
// y[:, :out_features] (reference: glq_output_rht_multiblock_kernel, glq/csrc/glq_cuda.cu:2151).
// FROM_F32: input is a plain fp32 (batch, m) matrix (the unfused output_rht op).
// ---------------------------------------------------------------------------------------------
template <bool FROM_F32>
__device__ __forceinline__ void rht_out_body(const DevLinear& L, const RhtItem it, const uint8_t* __restrict__ ws,
                                             uint8_t* __restrict__ y_base, const float* __restrict__ yrht_in,
                                             float* fbuf) {
  const int off = L.bm_off[it.block];
  const int logbs = L.bm_log[it.block];
  const int bs = 1 << logbs;
  const int rows_per_strip = (L.format == GLQB_FMT_TRELLIS_3INST) ? 32 : 16;
  const int m = L.m, fixed_slots = L.fixed_slots, gps = L.groups_per_strip, per_warp = L.per_warp;
  const long long slot_stride = (long long)L.batch * m;
  const float wscale = L.wscale;
  const float* row_scale = L.row_scale;
  const float* part = reinterpret_cast<const float*>(ws + L.part_off);
  auto slots_of = [&](int row) -> int {
    if (fixed_slots > 0) return fixed_slots;
    const long long g0 = L.group_base + (long long)(row / rows_per_strip) * gps;
    return (int)((g0 + gps - 1) / per_warp - g0 / per_warp) + 1;
  };
  auto load1 = [&](int trow, int i) -> float {
    const int row = off + i;
    const long long token = it.tok0 + trow;
    if constexpr (FROM_F32) return yrht_in[token * m + row];
    if (row >= m) return 0.f;
    const int cnt = slots_of(row);
    const float* p = part + token * m + row;
    float s = 0.f;
    for (int k = 0; k < cnt; ++k) s += __ldcg(p + k * slot_stride);
    s *= wscale;
    if (row_scale) s *= row_scale[row];
    return s;
  };
  if (L.stop_at_yrht) {            // rotated-domain result wanted: reduce and scale only
    const int total = it.ntok << logbs;
    for (int o = threadIdx.x; o < total; o += blockDim.x) {
      const int tk = o >> logbs, i = o & (bs - 1);
      if (off + i < m) reinterpret_cast<float*>(y_base)[L.y_off + (long long)(it.tok0 + tk) * L.y_stride + off + i] = load1(tk, i);
    }
    return;
  }
  const bool vec_ok = (m & 3) == 0 && (off & 3) == 0;
  const int tok0 = it.tok0;
  if (it.sub >= 0) {
    // split form: this CTA produces outputs [sub * 1024, sub * 1024 + 1024) of the block (see RhtItem::sub)
    const int S = bs >> RHT_SPLIT_LOG, k = it.sub;
    const float rs = rsqrtf((float)bs);
    for (int trow = 0; trow < it.ntok; ++trow) {
      // a fused RMSNorm of the single-launch kernel scales the output: its 1 / rms sits in the workspace
      const float in_scale = (L.in_norm_w && !L.xr_global) ? reinterpret_cast<const float*>(ws + L.rstd_off)[tok0 + trow] : 1.f;
      const long long o0 = L.y_off + (long long)(tok0 + trow) * L.y_stride + off + (k << RHT_SPLIT_LOG);
      auto ld1 = [&](int i) -> float {
        float a = 0.f;
        for (int kk = 0; kk < S; ++kk) {
          const float v = load1(trow, (kk << RHT_SPLIT_LOG) + i);
          a += (__popc(k & kk) & 1) ? -v : v;
        }
        return a * in_scale;
      };
      auto ld4 = [&](int i0, float (&q)[4]) {
#pragma unroll
        for (int j = 0; j < 4; ++j) q[j] = ld1(i0 + j);
      };
      const int r0 = off + (k << RHT_SPLIT_LOG);
      auto pre = [&](int i) -> float { return (r0 + i < L.out_f) ? __half2float(L.su[r0 + i]) : 0.f; };
      auto st = [&](int i, float val, float sign) {
        if (r0 + i < L.out_f) {
          float r = val * rs * sign;
          if (L.y_accumulate) r += load_act(y_base, o0 + i, L.y_dtype);
          store_act(y_base, o0 + i, L.y_dtype, r);
        }
      };
      fht_fast<RHT_SPLIT_LOG>(fbuf, RHT_SPLIT_LOG, ld1, ld4, pre, st);
      __syncthreads();
    }
    return;
  }
  if (blockDim.x == 256 && L.batch <= FUSED_MAX_TOKENS_C && gridDim.x <= RHT_LATENCY_MAX_ITEMS && logbs >= 5 && logbs <= RHT_FAST_MAX_LOG) {
    // decode-sized tile: the low-latency transform, token by token (see rht_in_body)
    const float rs = rsqrtf((float)bs);
    for (int trow = 0; trow < it.ntok; ++trow) {
      const long long o0 = L.y_off + (long long)(tok0 + trow) * L.y_stride + off;
      auto ld1 = [&](int i) -> float { return load1(trow, i); };
      auto ld4 = [&](int i0, float (&q)[4]) {
#pragma unroll
        for (int k = 0; k < 4; ++k) q[k] = load1(trow, i0 + k);
      };
      auto pre = [&](int i) -> float { return (off + i < L.out_f) ? __half2float(L.su[off + i]) : 0.f; };
      auto st = [&](int i, float val, float sign) {
        if (off + i < L.out_f) {
          float r = val * rs * sign;
          if (L.y_accumulate) r += load_act(y_base, o0 + i, L.y_dtype);
          store_act(y_base, o0 + i, L.y_dtype, r);
        }
      };
      fht_fast<RHT_FAST_MAX_LOG>(fbuf, logbs, ld1, ld4, pre, st);
      __syncthreads();
    }
    return;
  }
  auto load32 = [&](int trow, int i0, float (&v)[32]) {
    const int row0 = off + i0;
    const long long token = tok0 + trow;
    if (!vec_ok || row0 + 32 > m) {
#pragma unroll
      for (int k = 0; k < 32; ++k) v[k] = load1(trow, i0 + k);
      return;
    }
    const float* src = FROM_F32 ? (yrht_in + token * m + row0) : (part + token * m + row0);
    // the partial-sum count is a property of the strip (16 or 32 rows): two lookups cover the segment
    int cnt_lo = 1, cnt_hi = 1;
    if constexpr (!FROM_F32) { cnt_lo = slots_of(row0); cnt_hi = slots_of(row0 + 16); }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
      if constexpr (FROM_F32) {
        s = *reinterpret_cast<const float4*>(src + 4 * j);
      } else {
        const int cnt = j < 4 ? cnt_lo : cnt_hi;
        for (int k = 0; k < cnt; ++k) {
          const float4 t = __ldcg(reinterpret_cast<const float4*>(src + 4 * j + k * slot_stride));
          s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
        }
        s.x *= wscale; s.y *= wscale; s.z *= wscale; s.w *= wscale;
        if (row_scale) {
          const int r = row0 + 4 * j;
          s.x *= row_scale[r]; s.y *= row_scale[r + 1]; s.z *= row_scale[r + 2]; s.w *= row_scale[r + 3];
        }
      }
      v[4 * j] = s.x; v[4 * j + 1] = s.y; v[4 * j + 2] = s.z; v[4 * j + 3] = s.w;
    }
  };
  const float rs = rsqrtf((float)bs);
  const int out_f = L.out_f, y_dtype = L.y_dtype;
  const long long y_off = L.y_off, y_stride = L.y_stride;
  const __half* su = L.su;
  // 8 outputs per call: one 16-byte SU load and one 16-byte (32-byte for fp32) store when aligned
  const bool su_vec = (off & 7) == 0 && (reinterpret_cast<uintptr_t>(su) & 15) == 0;
  const bool y_vec = (reinterpret_cast<uintptr_t>(y_base) & 15) == 0;
  auto store8 = [&](int trow, int i0, const float (&v)[8], int count) {
    const int row0 = off + i0;
    const long long o = y_off + (long long)(tok0 + trow) * y_stride + row0;
    if (count == 8 && row0 + 8 <= out_f && su_vec && y_vec && (o & 7) == 0 && !L.y_accumulate) {
      const uint4 s4 = *reinterpret_cast<const uint4*>(su + row0);
      const float2 s0 = __half22float2(*reinterpret_cast<const __half2*>(&s4.x));
      const float2 s1 = __half22float2(*reinterpret_cast<const __half2*>(&s4.y));
      const float2 s2 = __half22float2(*reinterpret_cast<const __half2*>(&s4.z));
      const float2 s3 = __half22float2(*reinterpret_cast<const __half2*>(&s4.w));
      const float r[8] = {v[0] * rs * s0.x, v[1] * rs * s0.y, v[2] * rs * s1.x, v[3] * rs * s1.y,
                          v[4] * rs * s2.x, v[5] * rs * s2.y, v[6] * rs * s3.x, v[7] * rs * s3.y};
      if (y_dtype == GLQB_DT_F32) {
        float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(y_base) + o);
        dst[0] = make_float4(r[0], r[1], r[2], r[3]);
        dst[1] = make_float4(r[4], r[5], r[6], r[7]);
      } else if (y_dtype == GLQB_DT_F16) {
        const __half2 a = __floats2half2_rn(r[0], r[1]), b = __floats2half2_rn(r[2], r[3]);
        const __half2 c = __floats2half2_rn(r[4], r[5]), d = __floats2half2_rn(r[6], r[7]);
        *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(y_base) + o) =
            make_uint4(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b),
                       *reinterpret_cast<const uint32_t*>(&c), *reinterpret_cast<const uint32_t*>(&d));
      } else {
        const __nv_bfloat162 a = __floats2bfloat162_rn(r[0], r[1]), b = __floats2bfloat162_rn(r[2], r[3]);
        const __nv_bfloat162 c = __floats2bfloat162_rn(r[4], r[5]), d = __floats2bfloat162_rn(r[6], r[7]);
        *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(y_base) + o) =
            make_uint4(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b),
                       *reinterpret_cast<const uint32_t*>(&c), *reinterpret_cast<const uint32_t*>(&d));
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        if (k < count && row0 + k < out_f) {
          float r = v[k] * rs * __half2float(su[row0 + k]);
          if (L.y_accumulate) r += load_act(y_base, o + k, y_dtype);          // residual add
          store_act(y_base, o + k, y_dtype, r);
        }
    }
  };
  fht_tile8(fbuf, logbs, it.ntok, load32, load1, store8);
}

template <bool FROM_F32>
__global__ void __launch_bounds__(RHT_THREADS, GLQB_RHT_MINB) rht_out_kernel(const DevLinear* __restrict__ layers,
                                                              const RhtItem* __restrict__ items,
                                                              const uint8_t* __restrict__ ws,
                                                              uint8_t* __restrict__ y_base,
                                                              const float* __restrict__ yrht_in) {
  extern __shared__ float fbuf[];
  // launched with programmatic stream serialization behind the decode kernels: wait for them here; the next
  // kernel of the stream may start its prologue
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const RhtItem it = items[blockIdx.x];
  rht_out_body<FROM_F32>(layers[it.layer], it, ws, y_base, yrht_in, fbuf);
}

static __global__ void __launch_bounds__(RHT_THREADS, GLQB_RHT_MINB) rht_out_single_kernel(const __grid_constant__ DevLinear L,
                                                                     const __grid_constant__ RhtSingle S,
                                                                     uint8_t* __restrict__ y_base,
                                                                     const float* __restrict__ yrht_in) {
  extern __shared__ float fbuf[];
  rht_out_body<true>(L, rht_single_item(S, L.batch), nullptr, y_base, yrht_in, fbuf);
}

// ---------------------------------------------------------------------------------------------
// Trellis 3INST streaming decode + mma (batch <= 8*NB tokens ride the MMA columns).
//
// Work is the flattened list of 32x32 groups of every layer of the launch; warp w owns the
// contiguous range [w*per_warp, (w+1)*per_warp).  Inside a strip of 32 rows the warp accumulates in
// registers; at a strip boundary (or the end of its range) it writes one partial sum per
// (token, row) to slot (w - first warp touching the strip).  No atomics: the output transform adds
// the slots in ascending order, so results do not depend on scheduling.
//
// Per group and lane: one 4K-byte load of codes, K shuffles to fetch the next lane's chunks (the
// 16 bits that follow a lane's chunk in the tile's cyclic stream), one 16-byte load of rotated
// activations per 8 tokens, 32 state decodes, 4 MMAs per 8 tokens (two with a second stage).
// ---------------------------------------------------------------------------------------------
template <int K>
__device__ __forceinline__ Words<K> load_words(const uint8_t* p) {
  Words<K> v;
  if constexpr (K == 4) {
    uint4 t = ld_stream_v4(p); v.w[0] = t.x; v.w[1] = t.y; v.w[2] = t.z; v.w[3] = t.w;
  } else if constexpr (K == 2) {
    uint2 t = ld_stream_v2(p); v.w[0] = t.x; v.w[1] = t.y;
  } else if constexpr (K == 1) {
    v.w[0] = ld_stream_u32(p);
  } else {
    v.w[0] = ld_stream_u32(p); v.w[1] = ld_stream_u32(p + 4); v.w[2] = ld_stream_u32(p + 8);
  }
  return v;
}

template <int K>
__device__ __forceinline__ Words<K> shfl_words(const Words<K>& v, int src) {
  Words<K> r;
#pragma unroll
  for (int i = 0; i < K; ++i) r.w[i] = __shfl_sync(0xffffffffu, v.w[i], src);
  return r;
}

// decode the four tiles of a group and issue their MMAs against the B fragments xb[nb][ni]
// (xb[nb][ni] = {e0:(x,0) k-lo, e0 k-hi, e1 k-lo, e1 k-hi})
template <int K, int NB, int LUT = 0>
__device__ __forceinline__ void group_mma(const Words<K>& v, int lane, const uint4 (&xb)[NB][2],
                                          float (&acc)[NB][2][4], uint32_t lut_base = 0u) {
  const Words<K> vn = shfl_words<K>(v, (lane + 1) & 31);
  Words<K> vn2 = vn;
  if constexpr (K == 1) vn2 = shfl_words<K>(v, (lane + 2) & 31);
#pragma unroll
  for (int ni = 0; ni < 2; ++ni) {
#pragma unroll
    for (int mi = 0; mi < 2; ++mi) {
      const int q = ni * 2 + mi;
      uint32_t a[8];
      decode_tile<K, LUT>(chunk_of<K>(v, q), chunk_of<K>(vn, q), chunk_of<K>(vn2, q), a, lut_base);
      const uint32_t a_even[4] = {a[0], a[2], a[4], a[6]};   // columns 2t   / 8+2t   of the tile
      const uint32_t a_odd[4] = {a[1], a[3], a[5], a[7]};    // columns 2t+1 / 8+2t+1
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        mma16816(acc[nb][mi], a_even, xb[nb][ni].x, xb[nb][ni].y);
        mma16816(acc[nb][mi], a_odd, xb[nb][ni].z, xb[nb][ni].w);
      }
    }
  }
}

#ifndef GLQB_MINB
#define GLQB_MINB 3
#endif
// LUT > 0: the table form for large launches — one CTA of MV_LUT_THREADS per SM next to the 128 KiB table of the
// code's 65,536 fp16 values, which the CTA fills with the arithmetic decode when it starts (see decode_tile).
constexpr int MV_LUT_STATES = 2;
constexpr int MV_LUT_THREADS = GLQB_LUT_THREADS;
constexpr int MV_LUT_SMEM_BYTES = 65536 * 2;
template <int K1, int K2, int NB, int LUT = 0>
__global__ void __launch_bounds__(LUT ? MV_LUT_THREADS : MV_THREADS, LUT ? 1 : ((NB == 1 && K2 == 0) ? GLQB_MINB : 1))
trellis_mv_kernel(const DevLinear* __restrict__ layers, int n_layers, long long total_groups,
                  int per_warp, uint8_t* __restrict__ ws) {
  uint32_t lut_base = 0u;
  if constexpr (LUT > 0) {
    extern __shared__ __align__(16) unsigned short lut3[];
    for (int st = threadIdx.x; st < 65536; st += blockDim.x) lut3[st] = (unsigned short)(sum_dup3(hash3((uint32_t)st)) & 0xFFFFu);
    __syncthreads();
    lut_base = (uint32_t)__cvta_generic_to_shared(lut3);
  }
#ifndef GLQB_PF
#define GLQB_PF 4
#endif
  constexpr int PF = GLQB_PF;   // codes of PF groups in flight per lane
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  long long g = w * per_warp;
  const long long gend = min(g + per_warp, total_groups);
  if (g >= gend) return;
  // locate the layer holding group g (layers are sorted by group_base)
  int lo = 0, hi = n_layers - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (layers[mid].group_base <= g) lo = mid; else hi = mid - 1;
  }
  int li = lo;
  const int gq = lane >> 2, tq = lane & 3;

  while (g < gend) {
    const DevLinear& L = layers[li];
    const long long local = g - L.group_base;
    const int gps = L.groups_per_strip;
    const int strip = (int)(local / gps);
    const int c0 = (int)(local - (long long)strip * gps);
    const int c1 = (int)min((long long)gps, c0 + (gend - g));
    const int batch = L.batch;

    float acc[NB][2][4];
    float acc2[K2 ? NB : 1][2][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int i = 0; i < 4; ++i) { acc[nb][mi][i] = 0.f; if constexpr (K2 > 0) acc2[nb][mi][i] = 0.f; }

    const uint8_t* p1 = L.codes[0] + ((long long)strip * gps + c0) * (128 * K1) + lane * (4 * K1);
    const uint8_t* p2 = nullptr;
    if constexpr (K2 > 0) p2 = L.codes[1] + ((long long)strip * gps + c0) * (128 * K2) + lane * (4 * K2);
    const __half* xr = reinterpret_cast<const __half*>(ws + L.xr_off);
    // MMA column gq of block nb carries token 8*nb + gq.  Columns past the batch read the last
    // token again: their products land in accumulator columns that are never stored, which saves the
    // predicate and the zero fill on every group.
    const uint4* xq[NB];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int token = min(nb * 8 + gq, batch - 1);
      xq[nb] = reinterpret_cast<const uint4*>(xr + ((long long)token * L.n + c0 * 32) * XR_TRELLIS_EXPAND + tq * 16);
    }

    const int ng = c1 - c0;
    // One group step: codes of this group are in v/v2; the codes of the group PF ahead are requested
    // before the decode starts so that PF groups per lane are always in flight.
    Words<K1> cur[PF];
    Words<(K2 > 0 ? K2 : 1)> cur2[PF];
#pragma unroll
    for (int i = 0; i < PF; ++i) {
      if (i < ng) {
        cur[i] = load_words<K1>(p1 + i * (128 * K1));
        if constexpr (K2 > 0) cur2[i] = load_words<K2>(p2 + i * (128 * K2));
      }
    }
    const uint8_t* q1 = p1 + PF * (128 * K1);     // next codes to request
    const uint8_t* q2 = p2 + PF * (128 * K2);
    int c = 0;
    // full chunks with every prefetch in range: no per-group bounds checks
    for (; c + 2 * PF <= ng; c += PF) {
#pragma unroll
      for (int i = 0; i < PF; ++i) {
        const Words<K1> v = cur[i];
        Words<(K2 > 0 ? K2 : 1)> v2;
        if constexpr (K2 > 0) v2 = cur2[i];
        cur[i] = load_words<K1>(q1 + i * (128 * K1));
        if constexpr (K2 > 0) cur2[i] = load_words<K2>(q2 + i * (128 * K2));
        uint4 xb[NB][2];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          xb[nb][0] = __ldg(xq[nb] + i * 8);               // 64 halfs = 8 uint4 per group
          xb[nb][1] = __ldg(xq[nb] + i * 8 + 1);
        }
        group_mma<K1, NB, LUT>(v, lane, xb, acc, lut_base);
        if constexpr (K2 > 0) group_mma<K2, NB, LUT>(v2, lane, xb, acc2, lut_base);
      }
      q1 += PF * (128 * K1);
      q2 += PF * (128 * K2);
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) xq[nb] += PF * 8;
    }
    // tail: up to 2*PF - 1 groups, bounds checked
    for (; c < ng; c += PF) {
#pragma unroll
      for (int i = 0; i < PF; ++i) {
        if (c + i < ng) {
          const Words<K1> v = cur[i];
          Words<(K2 > 0 ? K2 : 1)> v2;
          if constexpr (K2 > 0) v2 = cur2[i];
          if (c + i + PF < ng) {
            cur[i] = load_words<K1>(q1 + i * (128 * K1));
            if constexpr (K2 > 0) cur2[i] = load_words<K2>(q2 + i * (128 * K2));
          }
          uint4 xb[NB][2];
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            xb[nb][0] = __ldg(xq[nb] + i * 8);
            xb[nb][1] = __ldg(xq[nb] + i * 8 + 1);
          }
          group_mma<K1, NB, LUT>(v, lane, xb, acc, lut_base);
          if constexpr (K2 > 0) group_mma<K2, NB, LUT>(v2, lane, xb, acc2, lut_base);
        }
      }
      q1 += PF * (128 * K1);
      q2 += PF * (128 * K2);
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) xq[nb] += PF * 8;
    }

    // flush: C fragment (row gq / gq+8, tokens 2tq, 2tq+1 of each column block)
    {
      const long long g0 = L.group_base + (long long)strip * gps;
      const int slot = (int)(w - g0 / per_warp);
      float* part = reinterpret_cast<float*>(ws + L.part_off) + (long long)slot * batch * L.m;
      const float s2 = L.stage_scale[1];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int token = nb * 8 + tq * 2 + (i & 1);
            const int row = strip * 32 + mi * 16 + gq + ((i >> 1) ? 8 : 0);
            if (token < batch) {
              float v = acc[nb][mi][i];
              if constexpr (K2 > 0) v = __fadd_rn(v, __fmul_rn(s2, acc2[nb][mi][i]));
              part[(long long)token * L.m + row] = v;
            }
          }
        }
      }
    }
    g += ng;
    if (c1 == gps && strip == L.strips - 1) ++li;
  }
}

// ---------------------------------------------------------------------------------------------
// One launch per decode linear (up to 8 tokens): input transform, 3INST decode + mma, output transform.
//
// Used for plans whose layers all read the same input (one layer, or the q/k/v / gate/up shards of a fused
// projection).  The reference's counterpart is its FUSE_IN matvec (glq/csrc/glq_trellis.cu:315-370, chosen at
// :1290-1295), which still needs a second launch for the output transform.
//   phase 1  every CTA recomputes the (cheap) input transform of the shared input into its own shared memory,
//            in the B-fragment layout of the MMAs — fht_tile, the same arithmetic as rht_in_kernel;
//   phase 2  work unit = (layer, 32-row strip, chunk of 64 column groups): warp w of the CTA decodes groups
//            [8w, 8w + 8) of the chunk; the eight warps' partial sums are added in warp order through shared
//            memory and written as partial sum number `chunk` of the strip (a strip of up to 2048 columns has
//            exactly one);
//   phase 3  a CTA that finishes the last unit of a Hadamard block of the output (integer ticket per block,
//            __threadfence before the increment; nobody ever waits) runs that block's output transform —
//            rht_out_body, the same arithmetic as rht_out_kernel.  The result does not depend on which CTA
//            that is.  Tickets are returned to zero by the CTA that completes them.
// ---------------------------------------------------------------------------------------------
constexpr int FUSED_CHUNK_GROUPS = 64;          // column groups per work unit: 8 warps x 8 groups
constexpr int FUSED_MAX_TOKENS = FUSED_MAX_TOKENS_C;
constexpr int FUSED_MAX_TODO = 32;

__device__ __forceinline__ uint4 lds_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}

// bytes of shared memory the transformed activations of a single-launch call take: trellis keeps (x, 0) half pairs
// in fragment order; E8 keeps fp16 in the order of xr_index_e8 (several tokens: interleaved in groups of eight)
template <bool E8FMT>
__host__ __device__ __forceinline__ size_t fused_xs_bytes(int n, int batch) {
  if (E8FMT) return (size_t)(batch == 1 ? 1 : 8) * n * 2;
  return (size_t)batch * n * 4;
}

// shared-memory bytes of the fused kernel: activations (2 halfs per column and token), transform scratch
// (the largest input block, or output tile, padded by one word per 32), the warps' partial sums
__host__ __device__ __forceinline__ size_t fused_smem_bytes(int n, int batch, int scratch_elems, bool e8 = false) {
  const size_t xs = e8 ? ((fused_xs_bytes<true>(n, batch) + 15) & ~(size_t)15) : fused_xs_bytes<false>(n, batch);
  return xs + ((size_t)scratch_elems + scratch_elems / 32) * 4 + 8 * 256 * 4 + 64;
}

// Output transform of one (layer, Hadamard block, token) by the CTA that completed the block, with the
// low-latency transform; same butterflies in the same order as rht_out_body, hence the same bits.  Blocks of up
// to 8192 rows (longer ones go through rht_out_body).
constexpr int FUSED_IN_MAX_LOG = 13;             // longest input block of the in-kernel shuffle transform: 8192
constexpr int FUSED_OUT_MAX_LOG = 13;            // longest output block the kernel can transform itself: 8192 (see out_split_log)

// `C` (tensor-parallel ranks, row-parallel layer): instead of being written to y, the block's transformed values are
// stored into every rank's receive area at float offset `piece` (this rank's source slot of epoch `comm_e`); the
// caller exchanges flags and adds the ranks' blocks afterwards.
__device__ __forceinline__ void fused_out_block(const DevLinear& L, int b, int tok, float in_scale,
                                                const uint8_t* __restrict__ ws, uint8_t* __restrict__ y_base, float* fbuf,
                                                const CommDev* C = nullptr, int comm_e = 0, long long piece = 0) {
  const int logbs = L.bm_log[b], off = L.bm_off[b];
  const int m = L.m, cnt = L.fixed_slots, out_f = L.out_f, y_dtype = L.y_dtype;
  const long long slot_stride = (long long)L.batch * m;
  const float wscale = L.wscale * in_scale;                  // in_scale: 1 / rms of the token (fused RMSNorm), else 1
  const float* row_scale = L.row_scale;
  const float* part = reinterpret_cast<const float*>(ws + L.part_off) + (long long)tok * m + off;
  auto load1 = [&](int i) -> float {
    float s = 0.f;
    for (int k = 0; k < cnt; ++k) s += __ldcg(part + i + k * slot_stride);
    s *= wscale;
    if (row_scale) s *= row_scale[off + i];
    return s;
  };
  auto load4 = [&](int i0, float (&q)[4]) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);

    for (int k = 0; k < cnt; ++k) {
      const float4 t = __ldcg(reinterpret_cast<const float4*>(part + i0 + k * slot_stride));
      s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
    }
    q[0] = s.x * wscale; q[1] = s.y * wscale; q[2] = s.z * wscale; q[3] = s.w * wscale;
    if (row_scale) {
#pragma unroll
      for (int k = 0; k < 4; ++k) q[k] *= row_scale[off + i0 + k];
    }
  };
  const long long yo = L.y_off + (long long)tok * L.y_stride + off;
  if (L.stop_at_yrht) {            // rotated-domain result wanted: reduce and scale only
    for (int i = threadIdx.x; i < (1 << logbs); i += blockDim.x) reinterpret_cast<float*>(y_base)[yo + i] = load1(i);
    return;
  }
  const float rs = rsqrtf((float)(1 << logbs));
  const __half* su = L.su + off;
  const bool accumulate = L.y_accumulate != 0;
  auto pre = [&](int i) -> float { return __half2float(su[i]); };      // the sign, requested before the partial sums
  auto store = [&](int i, float val, float sign) {
    if (off + i < out_f) {
      float r = val * rs * sign;
      if (accumulate) r += load_act(y_base, yo + i, y_dtype);          // residual add
      store_act(y_base, yo + i, y_dtype, r);
    }
  };
  if (C) {
    float* dst[COMM_MAX_RANKS];
#pragma unroll
    for (int r = 0; r < COMM_MAX_RANKS; ++r) dst[r] = r < C->world ? comm_slot(*C, r, comm_e, C->rank) + piece : nullptr;
    const int world = C->world;
    auto push = [&](int i, float val, float sign) {                    // consecutive threads, consecutive i
      const float r = val * rs * sign;
#pragma unroll
      for (int k = 0; k < COMM_MAX_RANKS; ++k)
        if (k < world) dst[k][i] = r;
    };
    fht_fast<FUSED_OUT_MAX_LOG>(fbuf, logbs, load1, load4, pre, push);
    return;
  }
  fht_fast<FUSED_OUT_MAX_LOG>(fbuf, logbs, load1, load4, pre, store);
}

// Phase 1 of the single-launch decode kernels: the transformed activations of the shared input, in shared memory
// (every CTA computes them itself; wide inputs are copied from the workspace, where rht_in_kernel left them).
// Fused RMSNorm: rstd_s[token] receives 1 / rms, which the callers apply to the OUTPUT.
template <bool E8FMT>
__device__ __forceinline__ void fused_phase1(const DevLinear& L0, int batch, const uint8_t* __restrict__ x_base,
                                             const uint8_t* __restrict__ ws, __half2* xs, float* fbuf, float* red,
                                             float* rstd_s) {
  const int n = L0.n;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (L0.xr_global) {
    // wide inputs: rht_in_kernel transformed them once, just before this kernel; every CTA copies the result
    const uint4* src = reinterpret_cast<const uint4*>(ws + L0.xr_off);
    uint4* dst = reinterpret_cast<uint4*>(xs);
    const int n16 = (int)(fused_xs_bytes<E8FMT>(n, batch) >> 4);
    for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = __ldcg(src + i);
    __syncthreads();
  } else {
    const int x_dtype = L0.x_dtype;
    const void* nw = L0.in_norm_w;
    const int nw_dtype = L0.in_norm_dtype;
    const bool gated = L0.in_gated_act != 0;
    const bool vec_ok = !gated && act_rows_aligned4(x_base, L0.x_off, L0.x_stride, x_dtype) &&
                        (nw == nullptr || (reinterpret_cast<uintptr_t>(nw) & 15) == 0);
    const __half* sv = L0.sv;
    for (int tok = 0; tok < batch; ++tok) {
      const long long xt0 = L0.x_off + (long long)tok * L0.x_stride;
      float ss = 0.f;                                        // this thread's share of sum(x^2) (fused RMSNorm)
      // value of column i_abs fed to the transform: x (or act(gate) * up), times the norm weight, times the sign.
      // The 1 / rms factor of the norm is a scalar per token and is applied to the output instead.
      auto load1 = [&](int i_abs) -> float {
        if (E8FMT && i_abs >= L0.in_f) return 0.f;           // padded E8 layers (trellis layers are never padded)
        float v = input_value(L0, x_base, xt0, i_abs);
        ss += v * v;
        if (nw) v *= load_act(nw, i_abs, nw_dtype);
        return v * __half2float(sv[i_abs]);
      };
      for (int b = 0; b < L0.nbn; ++b) {
        const int off = L0.bn_off[b], logbs = L0.bn_log[b];
        const float rs = rsqrtf((float)(1 << logbs));
        const bool vok = vec_ok && (off & 3) == 0;
        __half2* xt = xs + (size_t)tok * n;                  // trellis: n half2 per token, (x, 0) pairs in fragment order
        auto put = [&](int i, float val) {
          const int col = off + i;
          if constexpr (E8FMT) {
            reinterpret_cast<__half*>(xs)[xr_index_e8(tok, col, n, batch)] = __float2half_rn(val * rs);
          } else {
            xt[((col & ~31) * XR_TRELLIS_EXPAND + xr_pos_trellis(col & 31)) >> 1] =
                __halves2half2(__float2half_rn(val * rs), __float2half_rn(0.f));
          }
        };
        auto ld1 = [&](int i) -> float { return load1(off + i); };
        auto none = [](int) -> float { return 0.f; };
        auto put3 = [&](int i, float val, float) { put(i, val); };
        if (logbs <= FUSED_IN_MAX_LOG) {
          auto load4 = [&](int i0, float (&q)[4]) {
            if (vok && (!E8FMT || off + i0 + 3 < L0.in_f)) { // (padded E8 layers: columns past in_features read as zero)
              load_act4(x_base, xt0 + off + i0, x_dtype, q);
              ss += q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3];
              if (nw) {
                float w4[4];
                load_act4(nw, off + i0, nw_dtype, w4);
                q[0] *= w4[0]; q[1] *= w4[1]; q[2] *= w4[2]; q[3] *= w4[3];
              }
              const uint2 s4 = *reinterpret_cast<const uint2*>(sv + off + i0);
              const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&s4.x));
              const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&s4.y));
              q[0] *= a.x; q[1] *= a.y; q[2] *= c.x; q[3] *= c.y;
            } else {
#pragma unroll
              for (int k = 0; k < 4; ++k) q[k] = load1(off + i0 + k);
            }
          };
          fht_fast<FUSED_IN_MAX_LOG>(fbuf, logbs, ld1, load4, none, put3);
        } else {
          auto store1 = [&](int, int i, float val) { put(i, val); };
          auto l1 = [&](int, int i) -> float { return load1(off + i); };
          auto load32 = [&](int, int i0, float (&v)[32]) {
#pragma unroll
            for (int k = 0; k < 32; ++k) v[k] = load1(off + i0 + k);
          };
          fht_tile(fbuf, logbs, 1, load32, l1, store1);
        }
        __syncthreads();
      }
      if (nw) {                                              // every value of the token was loaded exactly once
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) red[warp] = ss;
        __syncthreads();
        if (threadIdx.x == 0) {
          float tot = 0.f;
          for (int w = 0; w < MV_WARPS; ++w) tot += red[w];
          rstd_s[tok] = rsqrtf(tot / (float)L0.in_f + L0.in_norm_eps);
        }
        __syncthreads();
      }
    }
  }

}

// Phase 3 of the single-launch decode kernels: output transforms of the blocks this CTA completed (`todo` entries
// are (layer << 8) | block), with the sum over tensor-parallel ranks when the layer asks for it.
__device__ __forceinline__ void fused_phase3(const DevLinear* layers, const int* todo, int nt, int batch, const float* rstd_s,
                                             const uint8_t* __restrict__ ws, uint8_t* __restrict__ y_base, float* fbuf,
                                             int scratch_elems, const CommDev& C, int comm_e) {
  for (int k = 0; k < nt; ++k) {
    const int li = todo[k] >> 8, b = todo[k] & 255;
    const DevLinear& L = layers[li];
    if (L.bm_log[b] <= FUSED_OUT_MAX_LOG) {
      if (C.world > 1 && L.reduce) {
        // Row-parallel layer: every rank transforms its own partial result (its own signs), stores the block into
        // all ranks' receive areas, and after the flag exchange adds the ranks' blocks in rank order: the same bits
        // on every rank, residual add included.
        const int logbs = L.bm_log[b], bs = 1 << logbs, off = L.bm_off[b];
        const long long piece = (long long)L.comm_off + (long long)off * batch;            // floats; a multiple of 32
        for (int tok = 0; tok < batch; ++tok) {
          fused_out_block(L, b, tok, rstd_s[tok], ws, y_base, fbuf, &C, comm_e, piece + ((long long)tok << logbs));
          __syncthreads();
        }
        comm_signal_and_wait(C, comm_e, L.comm_unit_base + b);
        const float* src = comm_slot(C, C.rank, comm_e, 0) + piece;
        const bool accumulate = L.y_accumulate != 0;
        for (int i = threadIdx.x * 4; i < bs * batch; i += blockDim.x * 4) {
          float4 a4 = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int r = 0; r < C.world; ++r) {
            const float4 t = __ldcg(reinterpret_cast<const float4*>(src + (size_t)r * C.max_floats + i));
            a4.x += t.x; a4.y += t.y; a4.z += t.z; a4.w += t.w;
          }
          const float o[4] = {a4.x, a4.y, a4.z, a4.w};
          const int tok = i >> logbs, j = i & (bs - 1);
          const long long yo = L.y_off + (long long)tok * L.y_stride + off + j;
#pragma unroll
          for (int c = 0; c < 4; ++c)
            if (off + j + c < L.out_f) {
              float r = o[c];
              if (accumulate) r += load_act(y_base, yo + c, L.y_dtype);
              store_act(y_base, yo + c, L.y_dtype, r);
            }
        }
        __syncthreads();
      } else {
        for (int tok = 0; tok < batch; ++tok) {
          fused_out_block(L, b, tok, rstd_s[tok], ws, y_base, fbuf);
          __syncthreads();
        }
      }
    } else {   // not reached: blocks longer than the split threshold are transformed by rht_out_kernel
      const int bs = 1 << L.bm_log[b];
      const int tt = max(1, min(batch, scratch_elems / bs));
      for (int t0 = 0; t0 < batch; t0 += tt) {
        rht_out_body<false>(L, RhtItem{li, b, t0, min(tt, batch - t0), -1}, ws, y_base, nullptr, fbuf);
        __syncthreads();
      }
    }
  }
}

#ifndef GLQB_FUSED_MINB
#define GLQB_FUSED_MINB 2
#endif
// The layers of a single-launch call travel in kernel-parameter space (constant bank): reading the plan's table
// from global memory would put several dependent L2 round trips at the head of a few-microsecond kernel.
constexpr int FUSED_MAX_LAYERS = 8;
struct FusedLayers {
  DevLinear L[FUSED_MAX_LAYERS];
};

template <int K1, int K2>
__global__ void __launch_bounds__(MV_THREADS, GLQB_FUSED_MINB)
trellis_fused_kernel(const __grid_constant__ FusedLayers T, int n_layers, int total_units, int scratch_elems,
                     const uint8_t* __restrict__ x_base, uint8_t* __restrict__ y_base, uint8_t* __restrict__ ws,
                     int* __restrict__ tickets, const __grid_constant__ CommDev C) {
  extern __shared__ __align__(16) uint8_t fsm[];
  const DevLinear* layers = T.L;
  const DevLinear& L0 = layers[0];
  const int n = L0.n, batch = L0.batch;
  __half2* xs = reinterpret_cast<__half2*>(fsm);                              // [batch][n] (x, 0) pairs, fragment order
  float* fbuf = reinterpret_cast<float*>(fsm + (size_t)batch * n * 4);
  float* red = fbuf + scratch_elems + scratch_elems / 32;                       // [8 warps][8 values][32 lanes]
  __shared__ int todo[FUSED_MAX_TODO];
  __shared__ int n_todo;
  if (threadIdx.x == 0) n_todo = 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, tq = lane & 3;

  // position of work unit u: layer, strip, chunk, this warp's first group and group count
  struct Unit { int li, strip, chunk, c0, ng; };
  auto locate = [&](int u) -> Unit {
    int li = 0;
    while (li + 1 < n_layers && layers[li + 1].group_base <= u) ++li;
    const DevLinear& L = layers[li];
    const int kch = L.fixed_slots;                          // chunks (= partial sums) per strip
    const int local = u - (int)L.group_base;
    const int strip = local / kch, chunk = local - strip * kch;
    const int gpw = L.per_warp;                             // column groups per warp and unit: 2, 4 or 8
    const int c0 = (chunk * MV_WARPS + warp) * gpw;
    return Unit{li, strip, chunk, c0, max(0, min(gpw, L.groups_per_strip - c0))};
  };
  // the stage-1 codes of a unit: all of a warp's (up to eight) groups in flight at once
  auto fetch = [&](const Unit& U, Words<K1> (&w1)[8]) {
    const DevLinear& L = layers[U.li];
    const uint8_t* p1 = L.codes[0] + ((long long)U.strip * L.groups_per_strip + U.c0) * (128 * K1) + lane * (4 * K1);
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (i < U.ng) w1[i] = load_words<K1>(p1 + i * (128 * K1));
  };

  // The codes do not depend on the activations: request the first unit's before the input transform, so the
  // trip to HBM overlaps it.
  int u = blockIdx.x;
  Unit U = locate(min(u, total_units - 1));
  Words<K1> w1[8];
  if (u < total_units) fetch(U, w1);
  // Programmatic dependent launch: let the next kernel of the stream start its own prologue, and wait here for
  // the previous kernel (which may have produced x) to finish.  Everything above reads only weights and the
  // plan's table.  Both are no-ops when the launch did not ask for the overlap.
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // tensor-parallel ranks (C.world > 1): the outputs are summed over the ranks inside this kernel (phase 3)
  const int comm_e = C.world > 1 ? comm_epoch(C) : 0;

  // ---- phase 1: the transformed activations of the shared input, in shared memory
  __shared__ float rstd_s[FUSED_MAX_TOKENS];                 // fused RMSNorm: 1 / rms per token, applied to the OUTPUT
  if (threadIdx.x < FUSED_MAX_TOKENS) rstd_s[threadIdx.x] = 1.f;
  fused_phase1<false>(L0, batch, x_base, ws, xs, fbuf, red, rstd_s);
  if (blockIdx.x == 0 && threadIdx.x < batch && L0.in_norm_w && !L0.xr_global)      // for rht_out_kernel (long blocks)
    for (int li = 0; li < n_layers; ++li) reinterpret_cast<float*>(ws + layers[li].rstd_off)[threadIdx.x] = rstd_s[threadIdx.x];

  // ---- phase 2: work units
  const uint32_t xs_addr = (uint32_t)__cvta_generic_to_shared(xs);
  while (u < total_units) {
    const DevLinear& L = layers[U.li];
    const int kch = L.fixed_slots, strip = U.strip, chunk = U.chunk, ng = U.ng, c0 = U.c0;
    const int gps = L.groups_per_strip;
    float acc[1][2][4], acc2[1][2][4];
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
      for (int i = 0; i < 4; ++i) { acc[0][mi][i] = 0.f; acc2[0][mi][i] = 0.f; }
    if (ng > 0) {
      Words<(K2 > 0 ? K2 : 1)> w2[8];
      if constexpr (K2 > 0) {
        const uint8_t* p2 = L.codes[1] + ((long long)strip * gps + c0) * (128 * K2) + lane * (4 * K2);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (i < ng) w2[i] = load_words<K2>(p2 + i * (128 * K2));
      }
      const int token = min(gq, batch - 1);                 // columns past the batch repeat the last token
      const uint32_t xa = xs_addr + (uint32_t)((((size_t)token * n + (size_t)c0 * 32) * XR_TRELLIS_EXPAND + tq * 16) * 2);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i < ng) {                                       // uniform per warp: the shuffles inside see all lanes
          uint4 xb[1][2];
          xb[0][0] = lds_v4(xa + i * 128);                  // 64 halfs = 128 bytes per group
          xb[0][1] = lds_v4(xa + i * 128 + 16);
          group_mma<K1, 1>(w1[i], lane, xb, acc);
          if constexpr (K2 > 0) group_mma<K2, 1>(w2[i], lane, xb, acc2);
        }
    }
    // next unit of this CTA: its codes travel while this one is reduced
    const int li_now = U.li;
    u += gridDim.x;
    if (u < total_units) { U = locate(u); fetch(U, w1); }
    {
      const float s2 = L.stage_scale[1];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float v = acc[0][mi][i];
          if constexpr (K2 > 0) v = __fadd_rn(v, __fmul_rn(s2, acc2[0][mi][i]));
          red[(warp * 8 + mi * 4 + i) * 32 + lane] = v;
        }
    }
    __syncthreads();
    {
      // thread (f, ln): fragment value f = mi * 4 + i of lane ln, summed over the warps in warp order
      const int f = threadIdx.x >> 5, ln = threadIdx.x & 31;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < MV_WARPS; ++w) s += red[(w * 8 + f) * 32 + ln];
      const int mi = f >> 2, i = f & 3;
      const int row = strip * 32 + mi * 16 + (ln >> 2) + ((i >> 1) ? 8 : 0);
      const int token = (ln & 3) * 2 + (i & 1);
      if (token < batch) reinterpret_cast<float*>(ws + L.part_off)[((long long)chunk * batch + token) * L.m + row] = s;
    }
    __syncthreads();                                        // the partial sums of the unit are written (and `red` is free)
    if (threadIdx.x == 0) {
      // which Hadamard block of the output holds this strip, and how many units make it complete
      int b = 0;
      while (b + 1 < L.nbm && strip * 32 >= L.bm_off[b + 1]) ++b;
      const int need = ((1 << L.bm_log[b]) >> 5) * kch;
      // release (the CTA's stores, ordered before this by the barrier) and acquire (the other CTAs' stores,
      // released before their increments) in one device-scope atomic; nobody ever waits on a ticket.
      // Long output blocks are left to rht_out_kernel, launched right behind this kernel: S CTAs share one there.
      int old = -2;
      if (L.bm_log[b] < L.out_split_log || L.stop_at_yrht)
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(tickets + L.ticket_base + b) : "memory");
      if (old + 1 == need) {
        tickets[L.ticket_base + b] = 0;                     // ready for the next run
        if (n_todo < FUSED_MAX_TODO) todo[n_todo++] = (li_now << 8) | b;
      }
    }
  }
  __syncthreads();

  // ---- phase 3: output transforms of the blocks this CTA completed
  fused_phase3(layers, todo, n_todo, batch, rstd_s, ws, y_base, fbuf, scratch_elems, C, comm_e);
  if (C.world > 1) comm_cta_done(C, comm_e);
}

// ---------------------------------------------------------------------------------------------
// E8 shell streaming gather + mma.
//
// Work group = 16 rows x 256 columns (32 indices per row).  Lane (g, t) loads 8 consecutive indices
// of row g and of row g+8 (columns 256*G + 64*t ...), gathers their nibble-packed codebook entries,
// expands each to 8 exact fp16 values and feeds two MMAs per index pair.  The MMA's k index is a
// dummy summation index, so a lane's 8 weights of one index may sit in any k slots as long as the
// activations are permuted the same way: the rotated activations are stored per 8-column block in
// the order (x0,x4,x1,x5,x2,x6,x3,x7), which lets a lane fetch the B fragments of both MMAs with
// one 16-byte load.  Every residual stage has its own accumulator (all stage values are exact in
// fp16); stages are combined in fp32 when a strip is flushed.
// ---------------------------------------------------------------------------------------------
// Where the codebook entries come from.  TM = 0: the packed tables stay in global memory (L1/L2
// gathers).  TM = 1: the first E8S_RESIDENT entries of the 65,536-entry table live in the CTA's shared
// memory (one CTA per SM) and are fetched with plain shared loads, bank conflicts and all; the few
// indices past the resident part still go to global memory.  Tables of up to 256 entries (the small
// second-stage codebook) are fully resident.
constexpr int E8S_RESIDENT = 56 * 1024;
struct E8Tables {
  uint32_t table_base;     // shared-window address of the resident part of the big table
  uint32_t small_base;     // shared-window address of the small table
};

// One stage's gather parameters, fixed per layer.
struct E8Stage {
  const uint32_t* table;   // global table
  uint32_t mask;           // entries - 1
  uint32_t base;           // TM = 1: shared-window address of the resident copy this stage indexes
};

// The gathers are volatile so that they keep their place ahead of the (volatile) MMAs of the chunk being
// consumed: that ordering is what keeps a whole chunk of gathers in flight.
template <int TM>
__device__ __forceinline__ uint32_t e8_gather(const E8Stage& S, uint32_t idx) {
  uint32_t v;
  const uint32_t* gp = S.table + idx;
  if constexpr (TM == 0) {
    asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(gp));
  } else {
    // branch-free: lanes whose index is resident read shared memory, the others global memory
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ge.u32 p, %1, %2;\n\t"
                 "@!p ld.shared.u32 %0, [%3];\n\t"
                 "@p ld.global.nc.u32 %0, [%4];\n\t}"
                 : "=r"(v)
                 : "r"(idx), "r"((uint32_t)E8S_RESIDENT), "r"(S.base + (idx << 2)), "l"(gp));
  }
  return v;
}

#ifndef GLQB_E8_KC
#define GLQB_E8_KC 8
#endif
#ifndef GLQB_E8_MINB
#define GLQB_E8_MINB 2
#endif
template <int NS, int NB, int TM>
__device__ __forceinline__ void e8_mv_body(const DevLinear* __restrict__ layers, int n_layers, long long total_groups,
                                           int per_warp, uint8_t* __restrict__ ws, const E8Tables& T,
                                           int warps_per_cta) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * warps_per_cta + (threadIdx.x >> 5);
  long long g = w * per_warp;
  const long long gend = min(g + per_warp, total_groups);
  if (g >= gend) return;
  int lo = 0, hi = n_layers - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (layers[mid].group_base <= g) lo = mid; else hi = mid - 1;
  }
  int li = lo;
  const int gq = lane >> 2, tq = lane & 3;

  while (g < gend) {
    const DevLinear& L = layers[li];
    const long long local = g - L.group_base;
    const int gps = L.groups_per_strip;
    const int strip = (int)(local / gps);
    const int c0 = (int)(local - (long long)strip * gps);
    const int c1 = (int)min((long long)gps, c0 + (gend - g));
    const int batch = L.batch;
    const int nidx = L.n >> 3;                 // indices per row
    bool vec_ok = (nidx & 7) == 0;             // rows (and the matrices themselves) start 16-byte aligned
#pragma unroll
    for (int s = 0; s < NS; ++s) vec_ok = vec_ok && (reinterpret_cast<uintptr_t>(L.codes[s]) & 15) == 0;
    const int rowA = strip * 16 + gq, rowB = rowA + 8;
    const bool okA = rowA < L.m, okB = rowB < L.m;

    float acc[NS][NB][4];
#pragma unroll
    for (int s = 0; s < NS; ++s)
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[s][nb][i] = 0.f;

    const __half* xr = reinterpret_cast<const __half*>(ws + L.xr_off);

    // Software pipeline over chunks of KC index pairs (a group is 8 / KC chunks).  While chunk cc is
    // expanded and multiplied, the codebook gathers of chunk cc+1 are in flight (KC * 2 * NS per lane)
    // and the index words of chunk cc+2 are on their way from HBM, so neither latency is exposed.
    constexpr int KC = (NS <= 2 && NB <= 2) ? GLQB_E8_KC : 4;
    constexpr int CPG = 8 / KC;
    constexpr int W = KC / 2;
    auto load_indices = [&](int cc, uint32_t (&qa)[NS][W], uint32_t (&qb)[NS][W]) {
      const int i0 = (cc / CPG) * 32 + tq * 8 + (cc % CPG) * KC;
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        const uint16_t* q = reinterpret_cast<const uint16_t*>(L.codes[s]);
        const uint16_t* pa = q + (long long)rowA * nidx + i0;
        const uint16_t* pb = q + (long long)rowB * nidx + i0;
        if (vec_ok && i0 + KC <= nidx) {
          if constexpr (KC == 8) {
            uint4 va = make_uint4(0, 0, 0, 0), vb = make_uint4(0, 0, 0, 0);
            if (okA) va = ld_stream_v4(pa);
            if (okB) vb = ld_stream_v4(pb);
            qa[s][0] = va.x; qa[s][1] = va.y; qa[s][2] = va.z; qa[s][3] = va.w;
            qb[s][0] = vb.x; qb[s][1] = vb.y; qb[s][2] = vb.z; qb[s][3] = vb.w;
          } else {
            uint2 va = make_uint2(0, 0), vb = make_uint2(0, 0);
            if (okA) va = ld_stream_v2(pa);
            if (okB) vb = ld_stream_v2(pb);
            qa[s][0] = va.x; qa[s][1] = va.y;
            qb[s][0] = vb.x; qb[s][1] = vb.y;
          }
        } else {
#pragma unroll
          for (int k = 0; k < W; ++k) {
            uint32_t a0 = 0, a1 = 0, b0 = 0, b1 = 0;
            if (i0 + 2 * k < nidx) { if (okA) a0 = pa[2 * k]; if (okB) b0 = pb[2 * k]; }
            if (i0 + 2 * k + 1 < nidx) { if (okA) a1 = pa[2 * k + 1]; if (okB) b1 = pb[2 * k + 1]; }
            qa[s][k] = a0 | (a1 << 16);
            qb[s][k] = b0 | (b1 << 16);
          }
        }
      }
    };
    E8Stage stg[NS];
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      stg[s].table = L.table[s];
      stg[s].mask = (uint32_t)L.table_entries[s] - 1u;
      stg[s].base = L.table_entries[s] == 65536 ? T.table_base : T.small_base;
    }
    auto gather = [&](const uint32_t (&qa)[NS][W], const uint32_t (&qb)[NS][W], uint32_t (&ea)[NS][KC],
                      uint32_t (&eb)[NS][KC]) {
#pragma unroll
      for (int s = 0; s < NS; ++s)
#pragma unroll
        for (int k = 0; k < KC; ++k) {
          ea[s][k] = e8_gather<TM>(stg[s], (qa[s][k >> 1] >> ((k & 1) * 16)) & stg[s].mask);
          eb[s][k] = e8_gather<TM>(stg[s], (qb[s][k >> 1] >> ((k & 1) * 16)) & stg[s].mask);
        }
    };
    // columns past the batch read the last token again (their accumulator columns are never stored)
    const uint4* xrow[NB];
    const int xstep = batch == 1 ? 1 : 8;      // 16-byte units between consecutive 8-column blocks
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int tok = min(nb * 8 + gq, batch - 1);
      xrow[nb] = reinterpret_cast<const uint4*>(xr) + (batch == 1 ? 0 : (long long)(tok >> 3) * nidx * 8 + (tok & 7));
    }
    auto consume = [&](int cc, const uint32_t (&ea)[NS][KC], const uint32_t (&eb)[NS][KC]) {
      const int i0 = (cc / CPG) * 32 + tq * 8 + (cc % CPG) * KC;   // first index (8-column block) of this lane
#pragma unroll
      for (int k = 0; k < KC; ++k) {
        const int blk = min(i0 + k, nidx - 1);
        uint4 xb[NB];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          xb[nb] = __ldg(xrow[nb] + blk * xstep);
          if (i0 + k >= nidx) xb[nb] = make_uint4(0u, 0u, 0u, 0u);   // past the row end: contributes nothing
        }
#pragma unroll
        for (int s = 0; s < NS; ++s) {
          uint32_t ha[4], hb[4];
          e8_entry_to_half2(ea[s][k], ha);
          e8_entry_to_half2(eb[s][k], hb);
          const uint32_t a1[4] = {ha[0], hb[0], ha[1], hb[1]};
          const uint32_t a2[4] = {ha[2], hb[2], ha[3], hb[3]};
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            mma16816(acc[s][nb], a1, xb[nb].x, xb[nb].y);
            mma16816(acc[s][nb], a2, xb[nb].z, xb[nb].w);
          }
        }
      }
    };

    const int cc0 = c0 * CPG, cc1 = c1 * CPG;
    uint32_t qa[NS][W], qb[NS][W];
    uint32_t eA[NS][KC], eB[NS][KC], fA[NS][KC], fB[NS][KC];
    load_indices(cc0, qa, qb);
    gather(qa, qb, eA, eB);
    if (cc0 + 1 < cc1) load_indices(cc0 + 1, qa, qb);
    for (int cc = cc0; cc < cc1; cc += 2) {
      if (cc + 1 < cc1) {
        gather(qa, qb, fA, fB);
        if (cc + 2 < cc1) load_indices(cc + 2, qa, qb);
      }
      consume(cc, eA, eB);
      if (cc + 1 < cc1) {
        if (cc + 2 < cc1) {
          gather(qa, qb, eA, eB);
          if (cc + 3 < cc1) load_indices(cc + 3, qa, qb);
        }
        consume(cc + 1, fA, fB);
      }
    }

    {
      const long long g0 = L.group_base + (long long)strip * gps;
      const int slot = (int)(w - g0 / per_warp);
      float* part = reinterpret_cast<float*>(ws + L.part_off) + (long long)slot * batch * L.m;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int token = nb * 8 + tq * 2 + (i & 1);
          const int row = (i >> 1) ? rowB : rowA;
          if (token < batch && row < L.m) {
            float v = acc[0][nb][i];
#pragma unroll
            for (int s = 1; s < NS; ++s) v = __fadd_rn(v, __fmul_rn(L.stage_scale[s], acc[s][nb][i]));
            part[(long long)token * L.m + row] = v;
          }
        }
      }
    }
    g += c1 - c0;
    if (c1 == gps && strip == L.strips - 1) ++li;
  }
}

template <int NS, int NB>
__global__ void __launch_bounds__(MV_THREADS, (NB <= 2 ? GLQB_E8_MINB : 1))
e8_mv_kernel(const DevLinear* __restrict__ layers, int n_layers, long long total_groups,
             int per_warp, uint8_t* __restrict__ ws) {
  const E8Tables T = {0u, 0u};
  e8_mv_body<NS, NB, 0>(layers, n_layers, total_groups, per_warp, ws, T, MV_WARPS);
}

// Resident-table form: one CTA per SM keeps most of the 65,536-entry table in shared memory.
#ifndef GLQB_E8S_THREADS
#define GLQB_E8S_THREADS 384
#endif
constexpr int E8S_THREADS = GLQB_E8S_THREADS;
constexpr int E8S_SMEM_BYTES = E8S_RESIDENT * 4 + 256 * 4;

template <int NS, int NB>
__global__ void __launch_bounds__(E8S_THREADS, 1)
e8_mv_smem_kernel(const DevLinear* __restrict__ layers, int n_layers, long long total_groups, int per_warp,
                  uint8_t* __restrict__ ws, const uint32_t* __restrict__ big_table,
                  const uint32_t* __restrict__ small_table, int small_entries) {
  extern __shared__ __align__(16) uint32_t e8_smem[];
  const uint4* src = reinterpret_cast<const uint4*>(big_table);
  uint4* dst = reinterpret_cast<uint4*>(e8_smem);
  for (int i = threadIdx.x; i < E8S_RESIDENT / 4; i += blockDim.x) dst[i] = __ldg(src + i);
  for (int i = threadIdx.x; i < small_entries && i < 256; i += blockDim.x) e8_smem[E8S_RESIDENT + i] = __ldg(small_table + i);
  E8Tables T;
  const uint32_t local = (uint32_t)__cvta_generic_to_shared(e8_smem);
  T.table_base = local;
  T.small_base = local + E8S_RESIDENT * 4;
  __syncthreads();
  e8_mv_body<NS, NB, 1>(layers, n_layers, total_groups, per_warp, ws, T, E8S_THREADS / 32);
}

// ---------------------------------------------------------------------------------------------
// Single-launch decode linear for E8-shell layers (at most 8 tokens, up to FUSED_MAX_LAYERS layers that read the
// same input): the same three phases as trellis_fused_kernel with the E8 streaming arithmetic in the middle.
// A work unit is (layer, 16-row strip, chunk of 8 warps x `per_warp` column groups of 256 columns); a lane (g, t)
// holds 8 consecutive indices of rows g and g + 8 per group and stage, gathers their packed table entries from
// global memory (L1 / L2: these launches are far too small to pay for a resident table), expands them with
// e8_entry_to_half2 and multiplies against the activations kept in shared memory in the order of xr_index_e8.
// Residual stages keep separate accumulators and are combined with fp32 multiply and add when the unit ends, as
// in e8_mv_body.  Replaces the three launches (input transform, matvec, output transform) of the reference's E8
// decode path (glq/csrc/glq_cuda.cu:2533, 3038) by one.
// ---------------------------------------------------------------------------------------------
constexpr int E8F_MAX_GPW = 4;                  // column groups per warp and unit (index registers: 8 per group)

// RES: the first `res_entries` entries of the 65,536-entry table (and a small second-stage table) are copied into
// shared memory at the start of the kernel — before the wait for the previous kernel, so the copy overlaps its tail
// — and one CTA runs per SM.  Used for launches of a few MB and more, where every SM would otherwise pull most of
// the table through L2 one 32-byte sector per gather (the launch's shared memory leaves too little L1 to hold it).
template <int NS, bool RES>
__global__ void __launch_bounds__(MV_THREADS, RES ? 1 : GLQB_FUSED_MINB)
e8_fused_kernel(const __grid_constant__ FusedLayers T, int n_layers, int total_units, int scratch_elems,
                const uint8_t* __restrict__ x_base, uint8_t* __restrict__ y_base, uint8_t* __restrict__ ws,
                int* __restrict__ tickets, const __grid_constant__ CommDev C, const uint32_t* __restrict__ big_table,
                int res_entries, const uint32_t* __restrict__ small_table, int small_entries) {
  extern __shared__ __align__(16) uint8_t fsm_all[];
  uint8_t* fsm = fsm_all + (RES ? (size_t)res_entries * 4 + 1024 : 0);
  const uint32_t table_smem = (uint32_t)__cvta_generic_to_shared(fsm_all);
  const uint32_t small_smem = table_smem + (uint32_t)res_entries * 4u;
  if constexpr (RES) {
    const uint4* src = reinterpret_cast<const uint4*>(big_table);
    uint4* dst = reinterpret_cast<uint4*>(fsm_all);
    for (int i = threadIdx.x; i < res_entries / 4; i += blockDim.x) dst[i] = __ldg(src + i);
    uint32_t* sm = reinterpret_cast<uint32_t*>(fsm_all + (size_t)res_entries * 4);
    for (int i = threadIdx.x; i < small_entries && i < 256; i += blockDim.x) sm[i] = __ldg(small_table + i);
  }
  const DevLinear* layers = T.L;
  const DevLinear& L0 = layers[0];
  const int n = L0.n, batch = L0.batch;
  __half2* xs = reinterpret_cast<__half2*>(fsm);
  float* fbuf = reinterpret_cast<float*>(fsm + ((fused_xs_bytes<true>(n, batch) + 15) & ~(size_t)15));
  float* red = fbuf + scratch_elems + scratch_elems / 32;                       // [8 warps][4 values][32 lanes]
  __shared__ int todo[FUSED_MAX_TODO];
  __shared__ int n_todo;
  if (threadIdx.x == 0) n_todo = 0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, tq = lane & 3;

  struct Unit { int li, strip, chunk, c0, ng; };
  auto locate = [&](int u) -> Unit {
    int li = 0;
    while (li + 1 < n_layers && layers[li + 1].group_base <= u) ++li;
    const DevLinear& L = layers[li];
    const int kch = L.fixed_slots;
    const int local = u - (int)L.group_base;
    const int strip = local / kch, chunk = local - strip * kch;
    const int gpw = L.per_warp;
    const int c0 = (chunk * MV_WARPS + warp) * gpw;
    return Unit{li, strip, chunk, c0, max(0, min(gpw, L.groups_per_strip - c0))};
  };
  // the indices of one stage of a unit: per group 8 of row g (qa) and 8 of row g + 8 (qb), 16 bytes each
  auto fetch = [&](const Unit& U, int stage, uint4 (&qa)[E8F_MAX_GPW], uint4 (&qb)[E8F_MAX_GPW]) {
    const DevLinear& L = layers[U.li];
    const int nidx = L.n >> 3;
    const uint16_t* q = reinterpret_cast<const uint16_t*>(L.codes[stage]);
    const int rowA = U.strip * 16 + gq, rowB = rowA + 8;
    const bool vec_ok = (nidx & 7) == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0;
#pragma unroll
    for (int i = 0; i < E8F_MAX_GPW; ++i) {
      qa[i] = make_uint4(0u, 0u, 0u, 0u);
      qb[i] = make_uint4(0u, 0u, 0u, 0u);
      if (i < U.ng) {
        const int i0 = (U.c0 + i) * 32 + tq * 8;
        const uint16_t* pa = q + (long long)rowA * nidx + i0;
        const uint16_t* pb = q + (long long)rowB * nidx + i0;
        if (vec_ok && i0 + 8 <= nidx) {
          if (rowA < L.m) qa[i] = ld_stream_v4(pa);
          if (rowB < L.m) qb[i] = ld_stream_v4(pb);
        } else {
          uint32_t wa[4] = {0u, 0u, 0u, 0u}, wb[4] = {0u, 0u, 0u, 0u};
#pragma unroll
          for (int k = 0; k < 8; ++k)
            if (i0 + k < nidx) {
              if (rowA < L.m) wa[k >> 1] |= (uint32_t)pa[k] << ((k & 1) * 16);
              if (rowB < L.m) wb[k >> 1] |= (uint32_t)pb[k] << ((k & 1) * 16);
            }
          qa[i] = make_uint4(wa[0], wa[1], wa[2], wa[3]);
          qb[i] = make_uint4(wb[0], wb[1], wb[2], wb[3]);
        }
      }
    }
  };

  // The indices do not depend on the activations: request the first unit's before the input transform.
  int u = blockIdx.x;
  Unit U = locate(min(u, total_units - 1));
  uint4 qa0[E8F_MAX_GPW], qb0[E8F_MAX_GPW];
  if (u < total_units) fetch(U, 0, qa0, qb0);
  asm volatile("griddepcontrol.launch_dependents;");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  const int comm_e = C.world > 1 ? comm_epoch(C) : 0;

  // ---- phase 1: the transformed activations of the shared input, in shared memory
  __shared__ float rstd_s[FUSED_MAX_TOKENS];
  if (threadIdx.x < FUSED_MAX_TOKENS) rstd_s[threadIdx.x] = 1.f;
  fused_phase1<true>(L0, batch, x_base, ws, xs, fbuf, red, rstd_s);
  if (blockIdx.x == 0 && threadIdx.x < batch && L0.in_norm_w && !L0.xr_global)
    for (int li = 0; li < n_layers; ++li) reinterpret_cast<float*>(ws + layers[li].rstd_off)[threadIdx.x] = rstd_s[threadIdx.x];

  // ---- phase 2: work units
  const uint32_t xs_addr = (uint32_t)__cvta_generic_to_shared(xs);
  const int nidx = n >> 3;
  // B fragments of one index (8-column block) for this lane's token: 16 bytes at block * xstep
  const int token = min(gq, batch - 1);                     // columns past the batch repeat the last token
  const uint32_t xa = xs_addr + (uint32_t)(batch == 1 ? 0 : (token & 7) * 16);
  const uint32_t xstep = batch == 1 ? 16u : 128u;
  while (u < total_units) {
    const DevLinear& L = layers[U.li];
    const int kch = L.fixed_slots, strip = U.strip, chunk = U.chunk, ng = U.ng, c0 = U.c0;
    float acc[NS][4];
#pragma unroll
    for (int st = 0; st < NS; ++st)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[st][i] = 0.f;
    if (ng > 0) {
#pragma unroll
      for (int st = 0; st < NS; ++st) {
        uint4 qa[E8F_MAX_GPW], qb[E8F_MAX_GPW];
        if (st > 0) fetch(U, st, qa, qb);
        const uint32_t* table = L.table[st];
        const uint32_t mask = (uint32_t)L.table_entries[st] - 1u;
        // resident form: big-table entries below res_entries and every small-table entry come from shared memory
        const bool is_big = L.table_entries[st] == 65536;
        const uint32_t sbase = is_big ? table_smem : small_smem;
        const uint32_t slimit = is_big ? (uint32_t)res_entries : 256u;
        auto gather = [&](uint32_t idx) -> uint32_t {
          if constexpr (RES) {
            uint32_t v;
            asm volatile("{\n\t.reg .pred p;\n\t"
                         "setp.ge.u32 p, %1, %2;\n\t"
                         "@!p ld.shared.u32 %0, [%3];\n\t"
                         "@p ld.global.nc.u32 %0, [%4];\n\t}"
                         : "=r"(v)
                         : "r"(idx), "r"(slimit), "r"(sbase + (idx << 2)), "l"(table + idx));
            return v;
          } else {
            return __ldg(table + idx);
          }
        };
#pragma unroll
        for (int i = 0; i < E8F_MAX_GPW; ++i) {
          if (i < ng) {
            const uint4 a4 = st == 0 ? qa0[i] : qa[i], b4 = st == 0 ? qb0[i] : qb[i];
            const uint32_t wa[4] = {a4.x, a4.y, a4.z, a4.w}, wb[4] = {b4.x, b4.y, b4.z, b4.w};
            uint32_t ea[8], eb[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {                   // all sixteen gathers of the group in flight
              ea[k] = gather((wa[k >> 1] >> ((k & 1) * 16)) & mask);
              eb[k] = gather((wb[k >> 1] >> ((k & 1) * 16)) & mask);
            }
            const int i0 = (c0 + i) * 32 + tq * 8;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const int blk = min(i0 + k, nidx - 1);
              uint4 xb = lds_v4(xa + (uint32_t)blk * xstep);
              if (i0 + k >= nidx) xb = make_uint4(0u, 0u, 0u, 0u);     // past the row end: contributes nothing
              uint32_t ha[4], hb[4];
              e8_entry_to_half2(ea[k], ha);
              e8_entry_to_half2(eb[k], hb);
              const uint32_t a1[4] = {ha[0], hb[0], ha[1], hb[1]};
              const uint32_t a2[4] = {ha[2], hb[2], ha[3], hb[3]};
              mma16816(acc[st], a1, xb.x, xb.y);
              mma16816(acc[st], a2, xb.z, xb.w);
            }
          }
        }
      }
    }
    // next unit of this CTA: its first-stage indices travel while this one is reduced
    const int li_now = U.li;
    u += gridDim.x;
    if (u < total_units) { U = locate(u); fetch(U, 0, qa0, qb0); }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float v = acc[0][i];
#pragma unroll
      for (int st = 1; st < NS; ++st) v = __fadd_rn(v, __fmul_rn(L.stage_scale[st], acc[st][i]));
      red[(warp * 4 + i) * 32 + lane] = v;
    }
    __syncthreads();
    if (threadIdx.x < 128) {
      // thread (f, ln): fragment value f of lane ln, summed over the warps in warp order
      const int f = threadIdx.x >> 5, ln = threadIdx.x & 31;
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < MV_WARPS; ++w) sum += red[(w * 4 + f) * 32 + ln];
      const int row = strip * 16 + (ln >> 2) + ((f >> 1) ? 8 : 0);
      const int tk = (ln & 3) * 2 + (f & 1);
      if (tk < batch && row < L.m) reinterpret_cast<float*>(ws + L.part_off)[((long long)chunk * batch + tk) * L.m + row] = sum;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int b = 0;
      while (b + 1 < L.nbm && strip * 16 >= L.bm_off[b + 1]) ++b;
      const int need = ((1 << L.bm_log[b]) >> 4) * kch;     // output blocks hold whole strips (16 rows or more)
      int old = -2;
      if (L.bm_log[b] < L.out_split_log || L.stop_at_yrht)
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(old) : "l"(tickets + L.ticket_base + b) : "memory");
      if (old + 1 == need) {
        tickets[L.ticket_base + b] = 0;
        if (n_todo < FUSED_MAX_TODO) todo[n_todo++] = (li_now << 8) | b;
      }
    }
  }
  __syncthreads();

  // ---- phase 3: output transforms of the blocks this CTA completed
  fused_phase3(layers, todo, n_todo, batch, rstd_s, ws, y_base, fbuf, scratch_elems, C, comm_e);
  if (C.world > 1) comm_cta_done(C, comm_e);
}

// ---------------------------------------------------------------------------------------------
// Dump kernels (bit-exact gate).  They call the same decode_tile / table expansion as the compute
// kernels and write the reconstructed rotated-domain weights in natural (row, col) order.
// ---------------------------------------------------------------------------------------------
template <int K1, int K2>
__global__ void __launch_bounds__(MV_THREADS)
trellis_dump_kernel(const uint8_t* __restrict__ p1, const uint8_t* __restrict__ p2, float s2,
                    int m, int n, void* __restrict__ out, int out_f32) {
  const int lane = threadIdx.x & 31;
  const int gps = n >> 5;
  const long long total = (long long)(m >> 5) * gps;
  for (long long g = (long long)blockIdx.x * MV_WARPS + (threadIdx.x >> 5); g < total;
       g += (long long)gridDim.x * MV_WARPS) {
    const int strip = (int)(g / gps), cp = (int)(g % gps);
    const Words<K1> v = load_words<K1>(p1 + g * (128 * K1) + lane * (4 * K1));
    const Words<K1> vn = shfl_words<K1>(v, (lane + 1) & 31);
    Words<K1> vn2 = vn;
    if constexpr (K1 == 1) vn2 = shfl_words<K1>(v, (lane + 2) & 31);
    Words<(K2 > 0 ? K2 : 1)> u, un, un2;
    if constexpr (K2 > 0) {
      u = load_words<K2>(p2 + g * (128 * K2) + lane * (4 * K2));
      un = shfl_words<K2>(u, (lane + 1) & 31);
      un2 = un;
      if constexpr (K2 == 1) un2 = shfl_words<K2>(u, (lane + 2) & 31);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int ni = q >> 1, mi = q & 1;
      uint32_t a[8], b[8];
      decode_tile<K1>(chunk_of<K1>(v, q), chunk_of<K1>(vn, q), chunk_of<K1>(vn2, q), a);
      if constexpr (K2 > 0) decode_tile<K2>(chunk_of<K2>(u, q), chunk_of<K2>(un, q), chunk_of<K2>(un2, q), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int row = strip * 32 + mi * 16 + tile_row(lane, j);
        const int col = cp * 32 + ni * 16 + tile_col(lane, j);
        const __half h = __ushort_as_half((unsigned short)(a[j] & 0xFFFFu));
        if (out_f32) {
          float f = __half2float(h);
          if constexpr (K2 > 0) {
            const __half h2 = __ushort_as_half((unsigned short)(b[j] & 0xFFFFu));
            f = __fadd_rn(f, __fmul_rn(__half2float(h2), s2));
          }
          reinterpret_cast<float*>(out)[(long long)row * n + col] = f;
        } else {
          reinterpret_cast<__half*>(out)[(long long)row * n + col] = h;
        }
      }
    }
  }
}

struct E8DumpArgs {
  const uint16_t* q[GLQB_MAX_STAGES];
  const uint32_t* table[GLQB_MAX_STAGES];
  int entries[GLQB_MAX_STAGES];
  float scale[GLQB_MAX_STAGES];
  int n_stages, m, n;
};

static __global__ void __launch_bounds__(256) e8_dump_kernel(E8DumpArgs A, float* __restrict__ out) {
  const int nidx = A.n >> 3;
  const long long total = (long long)A.m * nidx;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    float v[8];
    {
      const uint32_t e = A.table[0][A.q[0][i] & (uint32_t)(A.entries[0] - 1)];
      uint32_t h[4];
      e8_entry_to_half2(e, h);     // same expansion the matvec uses; unpack (c_k, c_{k+4})
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v[k] = __half2float(__ushort_as_half((unsigned short)(h[k] & 0xFFFFu)));
        v[k + 4] = __half2float(__ushort_as_half((unsigned short)(h[k] >> 16)));
      }
    }
    for (int s = 1; s < A.n_stages; ++s) {
      const uint32_t e = A.table[s][A.q[s][i] & (uint32_t)(A.entries[s] - 1)];
      uint32_t h[4];
      e8_entry_to_half2(e, h);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float lo = __half2float(__ushort_as_half((unsigned short)(h[k] & 0xFFFFu)));
        const float hi = __half2float(__ushort_as_half((unsigned short)(h[k] >> 16)));
        v[k] = __fadd_rn(v[k], __fmul_rn(lo, A.scale[s]));
        v[k + 4] = __fadd_rn(v[k + 4], __fmul_rn(hi, A.scale[s]));
      }
    }
    float* o = out + i * 8;
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = v[k];
  }
}

static __global__ void e8_pack_table_kernel(const __half* __restrict__ cb, int entries, uint32_t* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= entries) return;
  uint32_t p = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int code = __float2int_rn(__half2float(cb[i * 8 + k]) * 2.0f) + 6;
    p |= (uint32_t)(code & 0xF) << (4 * k);
  }
  out[i] = p;
}

}  // namespace glqb
