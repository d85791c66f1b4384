// MoE grouped expert matmul for trellis 3INST experts:
//     out[t] = sum_j w[t,j] * W2_e( act( W13_e x_t ) ),   e = topk_ids[t,j]
// (reference: glq_fused_moe_trellis_3inst_cuda, glq/csrc/glq_cuda.cu:5042; eager loop
// glq_vllm/fused_moe_method.py:393-440; storage glq_vllm/moe_shapes.py:56-72).
//
// Six launches (eight kernels and a memset from 8192 routings, see moe_launch_group), fixed grids, no host
// synchronisation (capture-safe):
//   1 moe_group_kernel     count tokens per expert, prefix sums, place every (token, j) routing in a slot
//                          (tensor-core form: also the per-expert layer entries and the GEMM work lists)
//   2 moe_rht_in_kernel    input transform of every TOKEN once (all experts share SV of w13)
//   3 trellis_moe_mv_kernel  w13: experts' weights decoded once per 8*NB routed tokens, partial sums per slot
//   4 moe_mid_kernel       a few slots per CTA: sum partials, Wscale, output transform, SU, gated activation,
//                          then the w2 input transform (SV, Hadamard) — three reference launches in one
//   5 trellis_moe_mv_kernel  w2
//   6 moe_out_kernel       per token: its routings are the rows of one tile transform; then, for j in fixed
//                          order, acc += w * SU * H(Wscale * partials)
// Work units of the two matmuls are (expert, 32-row strip, K chunk) and are handed out by an atomic
// counter, so skewed routing (a few hot experts) does not idle the warps that drew empty experts; the
// partial-sum slot of a unit is its K-chunk number, so results do not depend on which warp ran it.
// Integer atomics decide only WHERE a routing is stored, never a numeric value: outputs are
// bit-identical run to run.
//
// Steps with many routed tokens per expert take the tensor-core form instead: launches 3 and 5 become the
// tcgen05 GEMM kernel (glq_gemm_kernel, trellis producers) over a work list that the grouping kernel builds
// on the device from the expert counts — every expert is a "layer" whose token count, activation tiles and
// partial-sum rows are patched in each run; experts' routings are padded to whole 128-token tiles.  The
// transforms write the activations straight into the swizzled tile images the GEMM's bulk copies fetch.
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <vector>

#include "glqb_kernels.cuh"
#include "glqb_gemm.cuh"

namespace glqb {

struct MoeDev {
  // weights, expert-stacked
  const uint8_t* w13[2];
  const uint8_t* w2[2];
  long long w13_stride[2], w2_stride[2];   // bytes between experts
  const __half* w13_su; const __half* w13_sv; const float* w13_wscale; const float* w13_inv2;
  const __half* w2_su; const __half* w2_sv; const float* w2_wscale; const float* w2_inv2;
  int E, hidden, inter, w13_out, top_k, max_tokens, act, gated;
  int ids_i64, x_dtype, y_dtype;
  // Hadamard blocks: n13 (hidden), m13 (w13_out), n2 (inter), m2 (hidden)
  int nb_n13, nb_m13, nb_n2, nb_m2;
  int off_n13[GLQB_MAX_BLOCKS], log_n13[GLQB_MAX_BLOCKS];
  int off_m13[GLQB_MAX_BLOCKS], log_m13[GLQB_MAX_BLOCKS];
  int off_n2[GLQB_MAX_BLOCKS], log_n2[GLQB_MAX_BLOCKS];
  int off_m2[GLQB_MAX_BLOCKS], log_m2[GLQB_MAX_BLOCKS];
  // K chunking of the two matmuls
  int kch13, gpc13, kch2, gpc2;
  // workspace offsets (bytes)
  long long o_count, o_base, o_cursor, o_work, o_route_tok, o_route_exp, o_slot_of, o_xr1, o_part1, o_xr2, o_part2;
  // tensor-core form (gemm != 0): tile rows, device-built layer tables and work lists
  int gemm, k13a, k13b, k2a, k2b, max_items13, max_items2;
  long long o_trow, o_tile0, o_layers13, o_layers2, o_items13, o_items2, o_nitems, o_status;
  // E8 shell experts (format == GLQB_FMT_E8_SHELL; tensor-core form only): index matrices per stage,
  // expert-stacked, the packed tables, and the per-expert cumulative inverse residual scales of stages 2, 3
  int format, e8_ns;
  const uint8_t* e8_w13[3];
  const uint8_t* e8_w2[3];
  const uint32_t* e8_tab[3];
  int e8_ent[3];
  const float* e8_w13_inv[2];
  const float* e8_w2_inv[2];
};

constexpr int MOE_TN = 128;                    // routed tokens per GEMM tile
constexpr int MOE_B_BYTES = MOE_TN * 128;      // one 64-column chunk of a token tile

__device__ __forceinline__ float moe_act(float g, int act) {
  if (act == GLQB_ACT_SILU || act == 3) return g / (1.0f + __expf(-g));
  if (act == GLQB_ACT_GELU_TANH) {
    const float u = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.0f + tanhf(u));
  }
  if (act == 4) return 0.5f * g * (1.0f + erff(g * 0.7071067811865476f));     // gelu (exact), not gated
  const float r = fmaxf(g, 0.f);                                                 // relu^2 (codes 2 and 5)
  return r * r;
}

// ---- 1: grouping ------------------------------------------------------------------------------------
// phase 0: everything in this one CTA (small steps).  phase 1: the counts were made by moe_count_kernel and the
// routings are placed by moe_place_kernel (many CTAs each); this kernel only does the prefix sums and tables.
constexpr int MOE_GROUP_CHUNK = 8192;          // routings per CTA of the count / place kernels
constexpr int MOE_GROUP_SPLIT_MIN = 8192;      // routings from which the three-kernel form is used

__device__ __forceinline__ int moe_expert_of(const MoeDev& M, const void* ids, int i) {
  const long long v = M.ids_i64 ? reinterpret_cast<const long long*>(ids)[i] : (long long)reinterpret_cast<const int*>(ids)[i];
  return (v < 0 || v >= M.E) ? -1 : (int)v;
}

__global__ void __launch_bounds__(1024) moe_count_kernel(const __grid_constant__ MoeDev M, const void* __restrict__ ids,
                                                         int T, uint8_t* __restrict__ ws) {
  extern __shared__ int sh[];            // counts[E] of this CTA's chunk
  const int R = T * M.top_k;
  for (int e = threadIdx.x; e < M.E; e += blockDim.x) sh[e] = 0;
  __syncthreads();
  const int i0 = blockIdx.x * MOE_GROUP_CHUNK + threadIdx.x;
  int ev[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) { const int i = i0 + u * 1024; ev[u] = i < R ? moe_expert_of(M, ids, i) : -1; }
#pragma unroll
  for (int u = 0; u < 8; ++u) if (ev[u] >= 0) atomicAdd(&sh[ev[u]], 1);
  __syncthreads();
  int* g_count = reinterpret_cast<int*>(ws + M.o_count);
  for (int e = threadIdx.x; e < M.E; e += blockDim.x) if (sh[e]) atomicAdd(&g_count[e], sh[e]);
}

// Each CTA reserves, per expert, a contiguous run of slots for its chunk's routings (one global atomic per
// expert and CTA) and places them with shared-memory atomics.
__global__ void __launch_bounds__(1024) moe_place_kernel(const __grid_constant__ MoeDev M, const void* __restrict__ ids,
                                                         int T, uint8_t* __restrict__ ws) {
  extern __shared__ int sh[];            // counts[E], then cursor[E]
  int* cnt = sh;
  int* cur = sh + M.E;
  const int R = T * M.top_k;
  for (int e = threadIdx.x; e < M.E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  const int i0 = blockIdx.x * MOE_GROUP_CHUNK + threadIdx.x;
  int ev[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) { const int i = i0 + u * 1024; ev[u] = i < R ? moe_expert_of(M, ids, i) : -1; }
#pragma unroll
  for (int u = 0; u < 8; ++u) if (ev[u] >= 0) atomicAdd(&cnt[ev[u]], 1);
  __syncthreads();
  int* g_cursor = reinterpret_cast<int*>(ws + M.o_cursor);
  for (int e = threadIdx.x; e < M.E; e += blockDim.x) cur[e] = cnt[e] ? atomicAdd(&g_cursor[e], cnt[e]) : 0;
  __syncthreads();
  const int* g_base = reinterpret_cast<const int*>(ws + M.o_base);
  const int* g_tile0 = reinterpret_cast<const int*>(ws + M.o_tile0);
  int* route_tok = reinterpret_cast<int*>(ws + M.o_route_tok);
  int* route_exp = reinterpret_cast<int*>(ws + M.o_route_exp);
  int* slot_of = reinterpret_cast<int*>(ws + M.o_slot_of);
  int* trow = reinterpret_cast<int*>(ws + M.o_trow);
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const int i = i0 + u * 1024;
    if (i < R) {
      int slot = -1;
      if (ev[u] >= 0) {
        slot = atomicAdd(&cur[ev[u]], 1);
        route_tok[slot] = i / M.top_k;
        route_exp[slot] = ev[u];
        if (M.gemm) trow[slot] = g_tile0[ev[u]] * MOE_TN + (slot - g_base[ev[u]]);
      }
      slot_of[i] = slot;
    }
  }
}

__global__ void __launch_bounds__(1024) moe_group_kernel(const __grid_constant__ MoeDev M, const void* __restrict__ ids,
                                                         int T, uint8_t* __restrict__ ws, int phase) {
  extern __shared__ int sh[];            // counts[E], cursor[E], first slot[E], first token tile[E + 1]
  int* cnt = sh;
  int* cur = sh + M.E;
  int* base_s = sh + 2 * M.E;
  int* tile0 = sh + 3 * M.E;
  int* g_count = reinterpret_cast<int*>(ws + M.o_count);
  int* g_base = reinterpret_cast<int*>(ws + M.o_base);
  int* g_work = reinterpret_cast<int*>(ws + M.o_work);
  int* route_tok = reinterpret_cast<int*>(ws + M.o_route_tok);
  int* route_exp = reinterpret_cast<int*>(ws + M.o_route_exp);
  int* slot_of = reinterpret_cast<int*>(ws + M.o_slot_of);
  const int R = T * M.top_k;
  for (int e = threadIdx.x; e < M.E; e += blockDim.x) cnt[e] = 0;
  if (threadIdx.x < 2) g_work[threadIdx.x] = 0;
  __syncthreads();
  auto expert_of = [&](int i) -> int { return moe_expert_of(M, ids, i); };
  if (phase == 0) {
    // 8 routings per thread and round: the id loads of a round are issued together
    for (int i0 = threadIdx.x; i0 < R; i0 += 8 * blockDim.x) {
      int ev[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) { const int i = i0 + u * blockDim.x; ev[u] = i < R ? expert_of(i) : -1; }
#pragma unroll
      for (int u = 0; u < 8; ++u) if (ev[u] >= 0) atomicAdd(&cnt[ev[u]], 1);
    }
  } else {
    __syncthreads();
    for (int e = threadIdx.x; e < M.E; e += blockDim.x) cnt[e] = g_count[e];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, tiles = 0;
    for (int e = 0; e < M.E; ++e) {
      cur[e] = run; base_s[e] = run; run += cnt[e];
      tile0[e] = tiles; tiles += (cnt[e] + MOE_TN - 1) / MOE_TN;
    }
    tile0[M.E] = tiles;
  }
  __syncthreads();
  {
    int* g_cursor = reinterpret_cast<int*>(ws + M.o_cursor);
    int* g_tile0 = reinterpret_cast<int*>(ws + M.o_tile0);
    for (int e = threadIdx.x; e < M.E; e += blockDim.x) {
      g_base[e] = base_s[e]; g_count[e] = cnt[e]; g_cursor[e] = base_s[e]; g_tile0[e] = tile0[e];
    }
  }
  int* trow = reinterpret_cast<int*>(ws + M.o_trow);
  if (M.gemm) {
    // Tensor-core form.  Expert e with c routings owns ceil(c / 128) token tiles; routing number i of the
    // expert sits in row tile0[e] * 128 + i of the padded row space.  Every expert becomes a "layer" of the
    // GEMM kernel (token count, activation tiles and partial-sum rows of this step), and the work list is
    // ordered (token tile, row tile) so that the CTAs working at one moment share an activation tile in L2.
    const int kc13 = M.hidden / GM_TILE_K, kc2 = M.inter / GM_TILE_K;
    const int mt13 = (M.w13_out + GM_TILE_M - 1) / GM_TILE_M, mt2 = (M.hidden + GM_TILE_M - 1) / GM_TILE_M;
    const int tiles = tile0[M.E];
    if (threadIdx.x == 0) {
      int* nitems = reinterpret_cast<int*>(ws + M.o_nitems);
      nitems[0] = min(tiles * mt13, M.max_items13);
      nitems[1] = min(tiles * mt2, M.max_items2);
      reinterpret_cast<int*>(ws + M.o_status)[0] = 0;
    }
    DevLinear* L13 = reinterpret_cast<DevLinear*>(ws + M.o_layers13);
    DevLinear* L2 = reinterpret_cast<DevLinear*>(ws + M.o_layers2);
    for (int e = threadIdx.x; e < M.E; e += blockDim.x) {
      DevLinear a;
      memset(&a, 0, sizeof a);
      a.format = M.format;
      a.batch = cnt[e];
      DevLinear b = a;
      if (M.format == GLQB_FMT_E8_SHELL) {
        a.n_stages = b.n_stages = M.e8_ns;
        for (int s = 0; s < M.e8_ns; ++s) {
          a.codes[s] = M.e8_w13[s] + (long long)e * M.w13_stride[0];
          b.codes[s] = M.e8_w2[s] + (long long)e * M.w2_stride[0];
          a.table[s] = b.table[s] = M.e8_tab[s];
          a.table_entries[s] = b.table_entries[s] = M.e8_ent[s];
          a.stage_scale[s] = s ? M.e8_w13_inv[s - 1][e] : 1.f;
          b.stage_scale[s] = s ? M.e8_w2_inv[s - 1][e] : 1.f;
        }
      } else {
        a.codes[0] = M.w13[0] + (long long)e * M.w13_stride[0];
        a.codes[1] = M.w13[1] ? M.w13[1] + (long long)e * M.w13_stride[1] : nullptr;
        a.stage_scale[0] = 1.f; a.stage_scale[1] = M.w13_inv2 ? M.w13_inv2[e] : 0.f;
        b.codes[0] = M.w2[0] + (long long)e * M.w2_stride[0];
        b.codes[1] = M.w2[1] ? M.w2[1] + (long long)e * M.w2_stride[1] : nullptr;
        b.stage_scale[0] = 1.f; b.stage_scale[1] = M.w2_inv2 ? M.w2_inv2[e] : 0.f;
      }
      a.m = M.w13_out; a.n = M.hidden; a.strips = M.w13_out / 32; a.groups_per_strip = M.hidden / 32;
      a.xr_off = M.o_xr1 + (long long)tile0[e] * kc13 * MOE_B_BYTES;
      a.part_off = M.o_part1 + (long long)base_s[e] * M.w13_out * 4;
      b.m = M.hidden; b.n = M.inter; b.strips = M.hidden / 32; b.groups_per_strip = M.inter / 32;
      b.xr_off = M.o_xr2 + (long long)tile0[e] * kc2 * MOE_B_BYTES;
      b.part_off = M.o_part2 + (long long)base_s[e] * M.hidden * 4;
      L13[e] = a;
      L2[e] = b;
    }
    auto expert_of_tile = [&](int tile) -> int {       // last e with tile0[e] <= tile
      int lo = 0, hi = M.E - 1;
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (tile0[mid] <= tile) lo = mid; else hi = mid - 1;
      }
      return lo;
    };
    GemmItem* I13 = reinterpret_cast<GemmItem*>(ws + M.o_items13);
    GemmItem* I2 = reinterpret_cast<GemmItem*>(ws + M.o_items2);
    for (int idx = threadIdx.x; idx < min(tiles * mt13, M.max_items13); idx += blockDim.x) {
      const int tile = idx / mt13, e = expert_of_tile(tile);
      I13[idx] = GemmItem{e, idx - tile * mt13, tile - tile0[e], 0, kc13, 0};
    }
    for (int idx = threadIdx.x; idx < min(tiles * mt2, M.max_items2); idx += blockDim.x) {
      const int tile = idx / mt2, e = expert_of_tile(tile);
      I2[idx] = GemmItem{e, idx - tile * mt2, tile - tile0[e], 0, kc2, 0};
    }
  }
  if (phase != 0) return;
  for (int i0 = threadIdx.x; i0 < R; i0 += 8 * blockDim.x) {
    int ev[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) { const int i = i0 + u * blockDim.x; ev[u] = i < R ? expert_of(i) : -1; }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * blockDim.x;
      if (i < R) {
        int slot = -1;
        if (ev[u] >= 0) {
          slot = atomicAdd(&cur[ev[u]], 1);
          route_tok[slot] = i / M.top_k;
          route_exp[slot] = ev[u];
          if (M.gemm) trow[slot] = tile0[ev[u]] * MOE_TN + (slot - base_s[ev[u]]);
        }
        slot_of[i] = slot;
      }
    }
  }
}

// ---- 2: input transform per token (w13 side) -----------------------------------------------------------
__global__ void __launch_bounds__(1024) moe_rht_in_kernel(const __grid_constant__ MoeDev M, const uint8_t* __restrict__ x,
                                                          uint8_t* __restrict__ ws) {
  extern __shared__ float fb[];
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < M.hidden; i += blockDim.x)
    fb[i] = load_act(x, (long long)t * M.hidden + i, M.x_dtype) * __half2float(M.w13_sv[i]);
  for (int b = 0; b < M.nb_n13; ++b) fht_smem(fb + M.off_n13[b], M.log_n13[b]);
  __half2* out = reinterpret_cast<__half2*>(ws + M.o_xr1) + (long long)t * M.hidden;
  for (int b = 0; b < M.nb_n13; ++b) {
    const float rs = rsqrtf((float)(1 << M.log_n13[b]));
    for (int i = threadIdx.x; i < (1 << M.log_n13[b]); i += blockDim.x) {
      const int col = M.off_n13[b] + i;
      const int pos = (col & ~31) * XR_TRELLIS_EXPAND + xr_pos_trellis(col & 31);
      out[pos >> 1] = __halves2half2(__float2half_rn(fb[col] * rs), __float2half_rn(0.f));
    }
  }
}

// 16 bytes (8 consecutive columns starting at col8 * 8) of padded row `trow` in a [tile][chunk] x (128 x 64) image
__device__ __forceinline__ void moe_store_tile16(uint8_t* base, int trow, int kchunks, int col8, uint4 v) {
  const int tile = trow / MOE_TN, r = trow % MOE_TN;
  const int kc = col8 >> 3, e0 = (col8 & 7) * 8;
  *reinterpret_cast<uint4*>(base + ((size_t)tile * kchunks + kc) * MOE_B_BYTES + sw128_offset(r, e0)) = v;
}

__device__ __forceinline__ uint4 pack8_half(const float* f, float rs) {
  __half2 h0 = __floats2half2_rn(f[0] * rs, f[1] * rs), h1 = __floats2half2_rn(f[2] * rs, f[3] * rs);
  __half2 h2 = __floats2half2_rn(f[4] * rs, f[5] * rs), h3 = __floats2half2_rn(f[6] * rs, f[7] * rs);
  return make_uint4(*reinterpret_cast<uint32_t*>(&h0), *reinterpret_cast<uint32_t*>(&h1),
                    *reinterpret_cast<uint32_t*>(&h2), *reinterpret_cast<uint32_t*>(&h3));
}

// Input transform of one token, stored once per routing into the token tiles of the routed experts.
__global__ void __launch_bounds__(1024) moe_rht_in_gemm_kernel(const __grid_constant__ MoeDev M, const uint8_t* __restrict__ x,
                                                               uint8_t* __restrict__ ws) {
  extern __shared__ float fb[];
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < M.hidden; i += blockDim.x)
    fb[i] = load_act(x, (long long)t * M.hidden + i, M.x_dtype) * __half2float(M.w13_sv[i]);
  for (int b = 0; b < M.nb_n13; ++b) fht_smem(fb + M.off_n13[b], M.log_n13[b]);
  const int* slot_of = reinterpret_cast<const int*>(ws + M.o_slot_of);
  const int* trow = reinterpret_cast<const int*>(ws + M.o_trow);
  const int kchunks = M.hidden / GM_TILE_K;
  for (int b = 0; b < M.nb_n13; ++b) {
    const float rs = rsqrtf((float)(1 << M.log_n13[b]));
    for (int i = threadIdx.x * 8; i < (1 << M.log_n13[b]); i += blockDim.x * 8) {
      const int col = M.off_n13[b] + i;
      const uint4 v = pack8_half(fb + col, rs);
      for (int j = 0; j < M.top_k; ++j) {
        const int slot = slot_of[t * M.top_k + j];
        if (slot >= 0) moe_store_tile16(ws + M.o_xr1, trow[slot], kchunks, col >> 3, v);
      }
    }
  }
}

// ---- 3 / 5: grouped decode + mma ------------------------------------------------------------------------
struct MoeMvArgs {
  const uint8_t* codes[2];
  long long stride[2];
  const float* inv2;       // (E,) cumulative inverse residual scale of stage 2, or null
  const int* count;        // (E,)
  const int* base;         // (E,)
  const int* row_map;      // slot -> activation row, or null (identity)
  const __half* xr;        // activation rows, 2*n halfs each
  float* part;             // [kchunks][R][m]
  int* work;               // atomic unit counter
  int E, m, n, gps, strips, kchunks, gpc, R;
};

// One pass of a unit: the unit's groups are decoded once and multiplied with up to 8*NB routed tokens
// starting at t0.  Codes of MOE_PF groups are in flight per lane.
constexpr int MOE_PF = 4;

template <int K1, int K2, int NB>
__device__ __forceinline__ void moe_unit_pass(const MoeMvArgs& A, const uint8_t* p1, const uint8_t* p2, float s2, int ng,
                                              int c0, int strip, int kc, int base, int cnt, int t0, int lane) {
  const int gq = lane >> 2, tq = lane & 3;
  float acc[NB][2][4];
  float acc2[K2 ? NB : 1][2][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
      for (int i = 0; i < 4; ++i) { acc[nb][mi][i] = 0.f; if constexpr (K2 > 0) acc2[nb][mi][i] = 0.f; }
  const uint4* xq[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const int local = min(t0 + nb * 8 + gq, cnt - 1);     // columns past the count repeat the last token
    const int row = A.row_map ? A.row_map[base + local] : base + local;
    xq[nb] = reinterpret_cast<const uint4*>(A.xr + ((long long)row * A.n + c0 * 32) * XR_TRELLIS_EXPAND + tq * 16);
  }
  Words<K1> cur[MOE_PF];
  Words<(K2 > 0 ? K2 : 1)> cur2[MOE_PF];
#pragma unroll
  for (int i = 0; i < MOE_PF; ++i)
    if (i < ng) {
      cur[i] = load_words<K1>(p1 + i * (128 * K1));
      if constexpr (K2 > 0) cur2[i] = load_words<K2>(p2 + i * (128 * K2));
    }
  for (int c = 0; c < ng; c += MOE_PF) {
#pragma unroll
    for (int i = 0; i < MOE_PF; ++i) {
      if (c + i < ng) {
        const Words<K1> v = cur[i];
        Words<(K2 > 0 ? K2 : 1)> v2;
        if constexpr (K2 > 0) v2 = cur2[i];
        if (c + i + MOE_PF < ng) {
          cur[i] = load_words<K1>(p1 + (long long)(c + i + MOE_PF) * (128 * K1));
          if constexpr (K2 > 0) cur2[i] = load_words<K2>(p2 + (long long)(c + i + MOE_PF) * (128 * K2));
        }
        uint4 xb[NB][2];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          xb[nb][0] = __ldg(xq[nb] + (c + i) * 8);
          xb[nb][1] = __ldg(xq[nb] + (c + i) * 8 + 1);
        }
        group_mma<K1, NB>(v, lane, xb, acc);
        if constexpr (K2 > 0) group_mma<K2, NB>(v2, lane, xb, acc2);
      }
    }
  }
  float* part = A.part + (long long)kc * A.R * A.m;
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int local = t0 + nb * 8 + tq * 2 + (i & 1);
        const int row = strip * 32 + mi * 16 + gq + ((i >> 1) ? 8 : 0);
        if (local < cnt) {
          float v = acc[nb][mi][i];
          if constexpr (K2 > 0) v = __fadd_rn(v, __fmul_rn(s2, acc2[nb][mi][i]));
          part[(long long)(base + local) * A.m + row] = v;
        }
      }
}

// NBMAX = largest number of token-column blocks per pass (4 = 32 tokens; 2 with a second stage).  Every unit
// picks the smallest block count that covers its expert's tokens, so lightly loaded experts do not pay
// for MMAs on empty columns and heavily loaded ones are decoded once per 8*NBMAX tokens.
template <int K1, int K2, int NBMAX>
__global__ void __launch_bounds__(MV_THREADS, 2) trellis_moe_mv_kernel(const __grid_constant__ MoeMvArgs A) {
  const int lane = threadIdx.x & 31;
  const int units_per_expert = A.strips * A.kchunks;
  const int total_units = A.E * units_per_expert;
  // Every warp draws one unit at a time from an atomic counter (units of experts without tokens are
  // skipped at once, so skewed routing does not idle warps).
  for (;;) {
    int u = 0;
    if (lane == 0) u = atomicAdd(A.work, 1);
    u = __shfl_sync(0xffffffffu, u, 0);
    if (u >= total_units) break;
    const int e = u / units_per_expert;
    const int cnt = A.count[e];
    if (cnt == 0) continue;
    const int rem = u - e * units_per_expert;
    const int kc = rem / A.strips, strip = rem - kc * A.strips;
    const int c0 = kc * A.gpc, c1 = min(A.gps, c0 + A.gpc);
    const int base = A.base[e];
    const uint8_t* p1 = A.codes[0] + (long long)e * A.stride[0] + ((long long)strip * A.gps + c0) * (128 * K1) + lane * (4 * K1);
    const uint8_t* p2 = nullptr;
    float s2 = 0.f;
    if constexpr (K2 > 0) {
      p2 = A.codes[1] + (long long)e * A.stride[1] + ((long long)strip * A.gps + c0) * (128 * K2) + lane * (4 * K2);
      s2 = A.inv2[e];
    }
    const int ng = c1 - c0;
    int t0 = 0;
    for (; cnt - t0 > 8 * (NBMAX / 2); t0 += 8 * NBMAX)
      moe_unit_pass<K1, K2, NBMAX>(A, p1, p2, s2, ng, c0, strip, kc, base, cnt, t0, lane);
    if (cnt - t0 > 0) {
      if (NBMAX >= 4 && cnt - t0 > 8) moe_unit_pass<K1, K2, (NBMAX >= 4 ? 2 : 1)>(A, p1, p2, s2, ng, c0, strip, kc, base, cnt, t0, lane);
      else moe_unit_pass<K1, K2, 1>(A, p1, p2, s2, ng, c0, strip, kc, base, cnt, t0, lane);
    }
  }
}

// Shared-memory words of `rows` arrays laid out block after block, each array padded by one word per 32
// (the layout fht_tile works in): block b of row r starts at rows * pad_off[b] + r * row_words(b).
__device__ __forceinline__ int moe_pad_words(int n) { return n + (n >> 5); }

constexpr int MOE_XF_THREADS = 256;

// 8 fp16 values (16-byte aligned) as floats
__device__ __forceinline__ void load8_half(const __half* p, float (&f)[8]) {
  const uint4 t = *reinterpret_cast<const uint4*>(p);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t.x));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
  const float2 c = __half22float2(*reinterpret_cast<const __half2*>(&t.z));
  const float2 d = __half22float2(*reinterpret_cast<const __half2*>(&t.w));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ float round_half(float v) { return __half2float(__float2half_rn(v)); }

// ---- 4: per slot  h = act(gate) * up  from w13 partials, then the w2 input transform ---------------------
// One CTA handles `sg` consecutive slots (rows of the radix-32 tile transform).
__global__ void __launch_bounds__(MOE_XF_THREADS, 3) moe_mid_kernel(const __grid_constant__ MoeDev M, int T, int sg,
                                                                    uint8_t* __restrict__ ws) {
  extern __shared__ float fb[];              // sg x padded(max(w13_out, inter)) transform area, then sg x padded(inter)
  const int R = T * M.top_k;
  const int* g_count = reinterpret_cast<const int*>(ws + M.o_count);
  const int* g_base = reinterpret_cast<const int*>(ws + M.o_base);
  const int used = g_base[M.E - 1] + g_count[M.E - 1];
  const int slot0 = blockIdx.x * sg;
  if (slot0 >= used) return;
  const int nrow = min(sg, used - slot0);
  __shared__ int row_e[8];                   // expert of each row (sg <= 8)
  __shared__ float row_wsc[8];
  if (threadIdx.x < nrow) {
    const int e = reinterpret_cast<const int*>(ws + M.o_route_exp)[slot0 + threadIdx.x];
    row_e[threadIdx.x] = e;
    row_wsc[threadIdx.x] = M.w13_wscale[e];
  }
  __syncthreads();
  const int hrw = moe_pad_words(M.inter);
  float* hbuf = fb + sg * moe_pad_words(max(M.w13_out, M.inter));
  const float* part1 = reinterpret_cast<const float*>(ws + M.o_part1);
  const long long kstride = (long long)R * M.w13_out;
  const int kch = M.kch13, w13_out = M.w13_out, inter = M.inter;

  // -- output transform of w13 (Wscale applied on the way in); results stay in shared memory
  int poff = 0;
  for (int b = 0; b < M.nb_m13; ++b) {
    const int logbs = M.log_m13[b], off = M.off_m13[b];
    auto load32 = [&](int row, int i0, float (&v)[32]) {
      const float wsc = row_wsc[row];
      const float* src = part1 + (long long)(slot0 + row) * w13_out + off + i0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < kch; ++k) {
          const float4 t4 = *reinterpret_cast<const float4*>(src + 4 * j + k * kstride);
          a.x += t4.x; a.y += t4.y; a.z += t4.z; a.w += t4.w;
        }
        v[4 * j] = a.x * wsc; v[4 * j + 1] = a.y * wsc; v[4 * j + 2] = a.z * wsc; v[4 * j + 3] = a.w * wsc;
      }
    };
    fht_tile_core(fb + sg * poff, logbs, nrow, load32);
    poff += moe_pad_words(1 << logbs);
  }
  // -- 8 columns at a time: SU and 1/sqrt(bs), fp16 rounding (the reference's w13 op returns fp16:
  //    glq_vllm/fused_moe_method.py:412-421), gated activation, fp16 rounding, SV of w2
  auto y13_8 = [&](int row, int c, float (&f)[8]) {     // columns c .. c+7 of the w13 output (c % 8 == 0)
    int po = 0, b = 0;
    while (b + 1 < M.nb_m13 && c >= M.off_m13[b] + (1 << M.log_m13[b])) { po += moe_pad_words(1 << M.log_m13[b]); ++b; }
    const int bs = 1 << M.log_m13[b];
    const float rs = rsqrtf((float)bs);
    const float* p = fb + sg * po + row * moe_pad_words(bs) + fht_pad(c - M.off_m13[b]);
    float su[8];
    load8_half(M.w13_su + (long long)row_e[row] * w13_out + c, su);
#pragma unroll
    for (int k = 0; k < 8; ++k) f[k] = round_half(p[k] * rs * su[k]);
  };
  const int per_row = inter >> 3;
  for (int o = threadIdx.x; o < nrow * per_row; o += blockDim.x) {
    const int row = o / per_row, i = (o - row * per_row) * 8;
    float g[8], u[8], sv[8];
    y13_8(row, i, g);
    load8_half(M.w2_sv + i, sv);
    if (M.gated) y13_8(row, inter + i, u);
    float* dst = hbuf + row * hrw + fht_pad(i);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float a = moe_act(g[k], M.act);
      dst[k] = round_half(M.gated ? a * u[k] : a) * sv[k];
    }
  }
  __syncthreads();
  // -- input transform of w2, back into the transform area, then 16-byte stores
  poff = 0;
  for (int b = 0; b < M.nb_n2; ++b) {
    const int logbs = M.log_n2[b], off = M.off_n2[b];
    auto load32 = [&](int row, int i0, float (&v)[32]) {
      const float* src = hbuf + row * hrw + fht_pad(off + i0);    // off and i0 are multiples of 32
#pragma unroll
      for (int k = 0; k < 32; ++k) v[k] = src[k];
    };
    fht_tile_core(fb + sg * poff, logbs, nrow, load32);
    poff += moe_pad_words(1 << logbs);
  }
  poff = 0;
  const int* trow = reinterpret_cast<const int*>(ws + M.o_trow);
  for (int b = 0; b < M.nb_n2; ++b) {
    const int bs = 1 << M.log_n2[b], off = M.off_n2[b], rw = moe_pad_words(bs);
    const float* reg = fb + sg * poff;
    const float rs = rsqrtf((float)bs);
    const int pr = bs >> 3;
    for (int o = threadIdx.x; o < nrow * pr; o += blockDim.x) {
      const int row = o / pr, i = (o - row * pr) * 8;
      const float* src = reg + row * rw + fht_pad(i);
      const int slot = slot0 + row, col = off + i;
      if (M.gemm) {
        moe_store_tile16(ws + M.o_xr2, trow[slot], inter / GM_TILE_K, col >> 3, pack8_half(src, rs));
      } else {
        __half2* out = reinterpret_cast<__half2*>(ws + M.o_xr2) + (long long)slot * inter;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const int c = col + k;
          const int pos = (c & ~31) * XR_TRELLIS_EXPAND + xr_pos_trellis(c & 31);
          out[pos >> 1] = __halves2half2(__float2half_rn(src[k] * rs), __float2half_rn(0.f));
        }
      }
    }
    poff += rw;
  }
}

// ---- 6: per token weighted combine ------------------------------------------------------------------------
// The routings of a token are the rows of one tile transform (`rg` at a time); a thread then owns 8 output
// columns and adds the routings' results in fixed j order.
__global__ void __launch_bounds__(MOE_XF_THREADS, 3) moe_out_kernel(const __grid_constant__ MoeDev M, int T, int rg,
                                                                    const float* __restrict__ topk_w,
                                                                    const uint8_t* __restrict__ ws, uint8_t* __restrict__ y) {
  extern __shared__ float fb[];              // rg x padded(hidden) (+ hidden floats when several passes are needed)
  const int t = blockIdx.x;
  const int R = T * M.top_k;
  const int* slot_of = reinterpret_cast<const int*>(ws + M.o_slot_of);
  const int* route_exp = reinterpret_cast<const int*>(ws + M.o_route_exp);
  const float* part2 = reinterpret_cast<const float*>(ws + M.o_part2);
  __shared__ int row_slot[64], row_e[64];    // per routing j of this token (top_k <= 64)
  __shared__ float row_wsc[64], row_w[64];
  if (threadIdx.x < M.top_k) {
    const int slot = slot_of[t * M.top_k + threadIdx.x];
    const int e = slot >= 0 ? route_exp[slot] : 0;
    row_slot[threadIdx.x] = slot;
    row_e[threadIdx.x] = e;
    row_wsc[threadIdx.x] = M.w2_wscale[e];
    row_w[threadIdx.x] = topk_w[t * M.top_k + threadIdx.x];
  }
  __syncthreads();
  float* accs = fb + rg * moe_pad_words(M.hidden);   // running sums over the passes, hidden floats
  const int hidden = M.hidden, kch = M.kch2;
  const long long kstride = (long long)R * hidden;
  const bool y_vec = (reinterpret_cast<uintptr_t>(y) & 15) == 0;
  for (int j0 = 0; j0 < M.top_k; j0 += rg) {
    const int nrow = min(rg, M.top_k - j0);
    int poff = 0;
    for (int b = 0; b < M.nb_m2; ++b) {
      const int logbs = M.log_m2[b], off = M.off_m2[b];
      auto load32 = [&](int row, int i0, float (&v)[32]) {
        const int slot = row_slot[j0 + row];
        if (slot < 0) {
#pragma unroll
          for (int k = 0; k < 32; ++k) v[k] = 0.f;
          return;
        }
        const float wsc = row_wsc[j0 + row];
        const float* src = part2 + (long long)slot * hidden + off + i0;
#pragma unroll
        for (int jj = 0; jj < 8; ++jj) {
          float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int k = 0; k < kch; ++k) {
            const float4 t4 = *reinterpret_cast<const float4*>(src + 4 * jj + k * kstride);
            a.x += t4.x; a.y += t4.y; a.z += t4.z; a.w += t4.w;
          }
          v[4 * jj] = a.x * wsc; v[4 * jj + 1] = a.y * wsc; v[4 * jj + 2] = a.z * wsc; v[4 * jj + 3] = a.w * wsc;
        }
      };
      fht_tile_core(fb + rg * poff, logbs, nrow, load32);
      poff += moe_pad_words(1 << logbs);
    }
    const bool first = j0 == 0, last = j0 + rg >= M.top_k;
    for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
      int po = 0, b = 0;
      while (b + 1 < M.nb_m2 && c >= M.off_m2[b] + (1 << M.log_m2[b])) { po += moe_pad_words(1 << M.log_m2[b]); ++b; }
      const int bs = 1 << M.log_m2[b], rw = moe_pad_words(bs);
      const float rs = rsqrtf((float)bs);
      const float* reg = fb + rg * po + fht_pad(c - M.off_m2[b]);
      float a[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) a[k] = first ? 0.f : accs[c + k];
      for (int row = 0; row < nrow; ++row) {
        if (row_slot[j0 + row] < 0) continue;
        float su[8];
        load8_half(M.w2_su + (long long)row_e[j0 + row] * hidden + c, su);
        const float w = row_w[j0 + row];
        const float* p = reg + row * rw;
        // the reference's w2 op returns fp16 before the weighted sum
#pragma unroll
        for (int k = 0; k < 8; ++k) a[k] += w * round_half(p[k] * rs * su[k]);
      }
      if (!last) {
#pragma unroll
        for (int k = 0; k < 8; ++k) accs[c + k] = a[k];
      } else if (y_vec && M.y_dtype != GLQB_DT_F32) {
        uint4 o4;
        if (M.y_dtype == GLQB_DT_F16) {
          const __half2 h0 = __floats2half2_rn(a[0], a[1]), h1 = __floats2half2_rn(a[2], a[3]);
          const __half2 h2 = __floats2half2_rn(a[4], a[5]), h3 = __floats2half2_rn(a[6], a[7]);
          o4 = make_uint4(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1),
                          *reinterpret_cast<const uint32_t*>(&h2), *reinterpret_cast<const uint32_t*>(&h3));
        } else {
          const __nv_bfloat162 h0 = __floats2bfloat162_rn(a[0], a[1]), h1 = __floats2bfloat162_rn(a[2], a[3]);
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(a[4], a[5]), h3 = __floats2bfloat162_rn(a[6], a[7]);
          o4 = make_uint4(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1),
                          *reinterpret_cast<const uint32_t*>(&h2), *reinterpret_cast<const uint32_t*>(&h3));
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(y) + (long long)t * hidden + c) = o4;
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) store_act(y, (long long)t * hidden + c + k, M.y_dtype, a[k]);
      }
    }
    __syncthreads();
  }
}

typedef void (*MoeMvKernel)(const MoeMvArgs);

template <int NB>
static MoeMvKernel moe_mv_pick(int k1, int k2) {
#define M_CASE(A, B) if (k1 == A && k2 == B) return trellis_moe_mv_kernel<A, B, NB>;
  M_CASE(2, 0) M_CASE(3, 0) M_CASE(4, 0) M_CASE(4, 1) M_CASE(4, 2) M_CASE(4, 3) M_CASE(4, 4)
#undef M_CASE
  return nullptr;
}

typedef void (*MoeGemmKernel)(const DevLinear*, const GemmItem*, int, uint8_t*, int*, const int*);
constexpr int MOE_GEMM_STAGES = 4;
static MoeGemmKernel moe_gemm_pick(int k1, int k2) {
#define M_CASE(A, B) if (k1 == A && k2 == B) return glq_gemm_kernel<0, A, B, MOE_TN, MOE_GEMM_STAGES>;
  M_CASE(2, 0) M_CASE(3, 0) M_CASE(4, 0) M_CASE(4, 1) M_CASE(4, 2) M_CASE(4, 3) M_CASE(4, 4)
#undef M_CASE
  return nullptr;
}
static MoeGemmKernel moe_gemm_pick_e8(int ns) {
  switch (ns) {
    case 1: return glq_gemm_kernel<1, 1, 0, MOE_TN, MOE_GEMM_STAGES>;
    case 2: return glq_gemm_kernel<1, 2, 0, MOE_TN, MOE_GEMM_STAGES>;
    case 3: return glq_gemm_kernel<1, 3, 0, MOE_TN, MOE_GEMM_STAGES>;
  }
  return nullptr;
}
static size_t moe_gemm_smem_bytes() {
  return (size_t)MOE_GEMM_STAGES * (GM_A_BYTES + (size_t)MOE_B_BYTES) + (3 * MOE_GEMM_STAGES + 5) * 8 + 16 + 1024;
}
// routed tokens per expert (average) from which the tensor-core form is used
static int moe_gemm_min_avg() {
  const char* e = getenv("GLQB_MOE_GEMM_MIN_AVG");
  return e ? atoi(e) : 64;
}

}  // namespace glqb

using namespace glqb;

struct GlqbMoePlan {
  GlqbMoeDesc desc;
  MoeDev dev;
  size_t ws_bytes = 0;
  int sm_count = 0;
  int nb = 2;              // token-column blocks per pass (8*nb routed tokens share one decode)
  MoeMvKernel k13 = nullptr, k2 = nullptr;
  int grid13 = 0, grid2 = 0;
  int mid_sg = 1, out_rg = 1;          // slots per CTA of the mid kernel, routings per pass of the combine
  size_t mid_smem = 0, out_smem = 0;
  // tensor-core form
  bool gemm_ok = false;
  MoeDev devg;             // same weights, workspace laid out for the GEMM kernels
  MoeGemmKernel g13 = nullptr, g2 = nullptr;
  // optional timing of the two expert matmuls (event pairs around each, on the launching stream)
  bool timing = false;
  std::vector<cudaEvent_t> ev;
  size_t ev_used = 0;
};

// brackets one matmul launch with an event pair when timing is on
struct MoeTimer {
  GlqbMoePlan* P;
  cudaStream_t st;
  bool on;
  MoeTimer(GlqbMoePlan* p, cudaStream_t s) : P(p), st(s), on(p->timing) {
    if (!on) return;
    while (P->ev.size() < P->ev_used + 2) {
      cudaEvent_t e;
      if (cudaEventCreate(&e) != cudaSuccess) { on = false; return; }
      P->ev.push_back(e);
    }
    cudaEventRecord(P->ev[P->ev_used], st);
  }
  ~MoeTimer() {
    if (!on) return;
    cudaEventRecord(P->ev[P->ev_used + 1], st);
    P->ev_used += 2;
  }
};

static int moe_fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  set_error_message(buf);
  return code;
}

static size_t al(size_t v) { return (v + 255) / 256 * 256; }

static int fill_blocks(const int32_t* blocks, int nb, int total, int* off, int* lg, const char* what) {
  if (nb < 1 || nb > GLQB_MAX_BLOCKS) return moe_fail(GLQB_E_INVALID, "moe: %s block count %d", what, nb);
  int o = 0;
  for (int i = 0; i < nb; ++i) {
    const int b = blocks[i];
    if (b < 32 || (b & (b - 1))) return moe_fail(GLQB_E_INVALID, "moe: %s block %d", what, b);
    off[i] = o;
    lg[i] = 31 - __builtin_clz((unsigned)b);
    o += b;
  }
  if (o != total) return moe_fail(GLQB_E_INVALID, "moe: %s blocks sum to %d, expected %d", what, o, total);
  return GLQB_OK;
}

// grouping: one CTA for small steps; count / tables / place kernels (many CTAs) for large ones
static void moe_launch_group(const MoeDev& M, const void* ids, int tokens, uint8_t* ws, cudaStream_t st) {
  const int R = tokens * M.top_k;
  const size_t sh = (4 * (size_t)M.E + 1) * sizeof(int);
  if (R < MOE_GROUP_SPLIT_MIN) {
    moe_group_kernel<<<1, 1024, sh, st>>>(M, ids, tokens, ws, 0);
    return;
  }
  const int nb = (R + MOE_GROUP_CHUNK - 1) / MOE_GROUP_CHUNK;
  cudaMemsetAsync(ws + M.o_count, 0, sizeof(int) * M.E, st);
  moe_count_kernel<<<nb, 1024, M.E * sizeof(int), st>>>(M, ids, tokens, ws);
  moe_group_kernel<<<1, 1024, sh, st>>>(M, ids, tokens, ws, 1);
  moe_place_kernel<<<nb, 1024, 2 * M.E * sizeof(int), st>>>(M, ids, tokens, ws);
}

extern "C" {

int glqb_moe_plan_create(const GlqbMoeDesc* d, GlqbMoePlan** out) {
  if (!d || !out) return moe_fail(GLQB_E_INVALID, "moe_plan_create: null argument");
  if (d->num_experts < 1 || d->num_experts > 4096 || d->top_k < 1 || d->top_k > 64 || d->max_tokens < 1)
    return moe_fail(GLQB_E_INVALID, "moe_plan_create: experts=%d top_k=%d max_tokens=%d", d->num_experts, d->top_k,
                    d->max_tokens);
  const bool gated = d->activation >= 0 && d->activation <= 2;
  if (d->activation < 0 || d->activation > 5) return moe_fail(GLQB_E_INVALID, "moe_plan_create: activation %d", d->activation);
  const bool e8 = d->format == GLQB_FMT_E8_SHELL;
  if (d->format != GLQB_FMT_TRELLIS_3INST && !e8) return moe_fail(GLQB_E_INVALID, "moe_plan_create: format %d", d->format);
  if (d->hidden % 32 || d->inter % 32 || d->w13_out % 32)
    return moe_fail(GLQB_E_INVALID, "moe_plan_create: hidden/inter/w13_out must be multiples of 32");
  if (e8) {
    if (d->hidden % GM_TILE_K || d->inter % GM_TILE_K)
      return moe_fail(GLQB_E_INVALID, "moe_plan_create: E8 experts need hidden and inter to be multiples of 64");
    if (d->e8_stages < 1 || d->e8_stages > 3) return moe_fail(GLQB_E_INVALID, "moe_plan_create: E8 stages %d (1..3)", d->e8_stages);
    for (int s = 0; s < d->e8_stages; ++s) {
      const int en = d->e8_table_entries[s];
      if (!d->w13_qidxs[s] || !d->w2_qidxs[s] || !d->e8_table[s] || en < 1 || en > 65536 || (en & (en - 1)))
        return moe_fail(GLQB_E_INVALID, "moe_plan_create: E8 stage %d: null index matrix / table, or %d table entries", s, en);
      if (s && (!d->w13_inv_rs[s - 1] || !d->w2_inv_rs[s - 1]))
        return moe_fail(GLQB_E_INVALID, "moe_plan_create: E8 stage %d without its inverse residual scales", s);
    }
  }
  if (d->w13_out != (gated ? 2 : 1) * d->inter)
    return moe_fail(GLQB_E_INVALID, "moe_plan_create: w13_out=%d does not match inter=%d for activation %d", d->w13_out,
                    d->inter, d->activation);
  if (d->hidden > 8 * 1024 || d->inter > 4 * 1024 || d->w13_out > 16384)
    return moe_fail(GLQB_E_INVALID, "moe_plan_create: hidden <= 8192, inter <= 4096 supported");
  if ((!e8 && (!d->w13_packed || !d->w2_packed)) || !d->w13_su || !d->w13_sv || !d->w2_su || !d->w2_sv || !d->w13_wscale ||
      !d->w2_wscale)
    return moe_fail(GLQB_E_INVALID, "moe_plan_create: null weight pointer");
  if ((reinterpret_cast<uintptr_t>(d->w13_su) | reinterpret_cast<uintptr_t>(d->w13_sv) | reinterpret_cast<uintptr_t>(d->w2_su) |
       reinterpret_cast<uintptr_t>(d->w2_sv)) & 15)
    return moe_fail(GLQB_E_INVALID, "moe_plan_create: SU/SV tensors must be 16-byte aligned");
  GlqbMoePlan* P = new GlqbMoePlan();
  P->desc = *d;
  MoeDev& M = P->dev;
  memset(&M, 0, sizeof M);
  int rc;
  if ((rc = fill_blocks(d->blocks_n_w13, d->n_blocks_n_w13, d->hidden, M.off_n13, M.log_n13, "n_w13")) ||
      (rc = fill_blocks(d->blocks_m_w13, d->n_blocks_m_w13, d->w13_out, M.off_m13, M.log_m13, "m_w13")) ||
      (rc = fill_blocks(d->blocks_n_w2, d->n_blocks_n_w2, d->inter, M.off_n2, M.log_n2, "n_w2")) ||
      (rc = fill_blocks(d->blocks_m_w2, d->n_blocks_m_w2, d->hidden, M.off_m2, M.log_m2, "m_w2"))) {
    delete P;
    return rc;
  }
  M.nb_n13 = d->n_blocks_n_w13; M.nb_m13 = d->n_blocks_m_w13; M.nb_n2 = d->n_blocks_n_w2; M.nb_m2 = d->n_blocks_m_w2;
  // E8 experts run the tensor-core form at every token count; the streaming kernels below are picked with
  // placeholder rates and never launched for them
  const int k13a = e8 ? 4 : d->w13_bits, k13b = (!e8 && d->w13_packed2) ? d->w13_bits2 : 0;
  const int k2a = e8 ? 4 : d->w2_bits, k2b = (!e8 && d->w2_packed2) ? d->w2_bits2 : 0;
  // tokens per decode pass: 16 for small steps, 32 when experts see many tokens
  const double avg = (double)d->max_tokens * d->top_k / d->num_experts;
  (void)avg;
  P->nb = (k13b || k2b) ? 2 : 4;
  P->k13 = P->nb == 4 ? moe_mv_pick<4>(k13a, k13b) : moe_mv_pick<2>(k13a, k13b);
  P->k2 = P->nb == 4 ? moe_mv_pick<4>(k2a, k2b) : moe_mv_pick<2>(k2a, k2b);
  if (!P->k13 || !P->k2) {
    delete P;
    return moe_fail(GLQB_E_INVALID, "moe_plan_create: no kernel for trellis rates w13 K=%d+%d, w2 K=%d+%d", k13a, k13b, k2a,
                    k2b);
  }
  M.w13[0] = (const uint8_t*)d->w13_packed; M.w13[1] = (const uint8_t*)d->w13_packed2;
  M.w2[0] = (const uint8_t*)d->w2_packed; M.w2[1] = (const uint8_t*)d->w2_packed2;
  M.w13_stride[0] = (long long)d->w13_out * d->hidden * k13a / 8;
  M.w13_stride[1] = (long long)d->w13_out * d->hidden * k13b / 8;
  M.w2_stride[0] = (long long)d->hidden * d->inter * k2a / 8;
  M.w2_stride[1] = (long long)d->hidden * d->inter * k2b / 8;
  M.format = d->format;
  if (e8) {
    M.e8_ns = d->e8_stages;
    M.w13_stride[0] = (long long)d->w13_out * (d->hidden / 8) * 2;     // int16 per 8 weights, every stage
    M.w2_stride[0] = (long long)d->hidden * (d->inter / 8) * 2;
    M.w13_stride[1] = M.w2_stride[1] = 0;
    for (int s = 0; s < d->e8_stages; ++s) {
      M.e8_w13[s] = (const uint8_t*)d->w13_qidxs[s];
      M.e8_w2[s] = (const uint8_t*)d->w2_qidxs[s];
      M.e8_tab[s] = d->e8_table[s];
      M.e8_ent[s] = d->e8_table_entries[s];
      if (s) { M.e8_w13_inv[s - 1] = d->w13_inv_rs[s - 1]; M.e8_w2_inv[s - 1] = d->w2_inv_rs[s - 1]; }
    }
  }
  M.w13_su = (const __half*)d->w13_su; M.w13_sv = (const __half*)d->w13_sv;
  M.w13_wscale = d->w13_wscale; M.w13_inv2 = d->w13_inv_resid_scale2;
  M.w2_su = (const __half*)d->w2_su; M.w2_sv = (const __half*)d->w2_sv;
  M.w2_wscale = d->w2_wscale; M.w2_inv2 = d->w2_inv_resid_scale2;
  if ((k13b && !M.w13_inv2) || (k2b && !M.w2_inv2)) {
    delete P;
    return moe_fail(GLQB_E_INVALID, "moe_plan_create: second stage without its inverse residual scales");
  }
  M.E = d->num_experts; M.hidden = d->hidden; M.inter = d->inter; M.w13_out = d->w13_out; M.top_k = d->top_k;
  M.max_tokens = d->max_tokens; M.act = d->activation; M.gated = gated ? 1 : 0;
  M.ids_i64 = d->ids_are_int64; M.x_dtype = d->x_dtype; M.y_dtype = d->y_dtype;
  // K chunking: 32 groups (1024 columns) per unit
  const int gps13 = d->hidden / 32, gps2 = d->inter / 32;
  M.gpc13 = std::min(gps13, 32); M.kch13 = (gps13 + M.gpc13 - 1) / M.gpc13;
  M.gpc2 = std::min(gps2, 32); M.kch2 = (gps2 + M.gpc2 - 1) / M.gpc2;
  // workspace
  const size_t R = (size_t)d->max_tokens * d->top_k;
  size_t o = 0;
  M.o_count = o; o = al(o + 4 * (size_t)M.E);
  M.o_base = o; o = al(o + 4 * (size_t)M.E);
  M.o_cursor = o; o = al(o + 4 * (size_t)M.E);
  M.o_tile0 = o; o = al(o + 4 * ((size_t)M.E + 1));
  M.o_work = o; o = al(o + 16);
  M.o_route_tok = o; o = al(o + 4 * R);
  M.o_route_exp = o; o = al(o + 4 * R);
  M.o_slot_of = o; o = al(o + 4 * R);
  M.o_xr1 = o; o = al(o + (size_t)d->max_tokens * d->hidden * 2 * XR_TRELLIS_EXPAND);
  M.o_part1 = o; o = al(o + (size_t)M.kch13 * R * d->w13_out * 4);
  M.o_xr2 = o; o = al(o + R * d->inter * 2 * XR_TRELLIS_EXPAND);
  M.o_part2 = o; o = al(o + (size_t)M.kch2 * R * d->hidden * 4);
  P->ws_bytes = o;
  // tensor-core form: its buffers overlay the decode form's (a step runs one or the other)
  P->g13 = e8 ? moe_gemm_pick_e8(d->e8_stages) : moe_gemm_pick(k13a, k13b);
  P->g2 = e8 ? moe_gemm_pick_e8(d->e8_stages) : moe_gemm_pick(k2a, k2b);
  P->gemm_ok = P->g13 && P->g2 && d->hidden % GM_TILE_K == 0 && d->inter % GM_TILE_K == 0 && M.E <= 4096 &&
               (e8 || R >= (size_t)M.E * moe_gemm_min_avg());
  if (P->gemm_ok) {
    MoeDev& G = P->devg;
    G = M;
    G.gemm = 1; G.kch13 = 1; G.kch2 = 1;
    G.k13a = k13a; G.k13b = k13b; G.k2a = k2a; G.k2b = k2b;
    const size_t tiles = R / MOE_TN + M.E;
    const size_t mt13 = (d->w13_out + GM_TILE_M - 1) / GM_TILE_M, mt2 = (d->hidden + GM_TILE_M - 1) / GM_TILE_M;
    G.max_items13 = (int)(tiles * mt13);
    G.max_items2 = (int)(tiles * mt2);
    auto al1k = [](size_t v) { return (v + 1023) / 1024 * 1024; };
    size_t g = al1k((size_t)M.o_xr1);
    G.o_xr1 = g; g = al1k(g + tiles * (d->hidden / GM_TILE_K) * MOE_B_BYTES);
    G.o_part1 = g; g = al1k(g + R * d->w13_out * 4);
    G.o_xr2 = g; g = al1k(g + tiles * (d->inter / GM_TILE_K) * MOE_B_BYTES);
    G.o_part2 = g; g = al1k(g + R * d->hidden * 4);
    G.o_trow = g; g = al1k(g + 4 * R);
    G.o_layers13 = g; g = al1k(g + sizeof(DevLinear) * M.E);
    G.o_layers2 = g; g = al1k(g + sizeof(DevLinear) * M.E);
    G.o_items13 = g; g = al1k(g + sizeof(GemmItem) * G.max_items13);
    G.o_items2 = g; g = al1k(g + sizeof(GemmItem) * G.max_items2);
    G.o_nitems = g; g = al1k(g + 16);
    G.o_status = g; g = al1k(g + 16);
    P->ws_bytes = std::max(P->ws_bytes, g);
    if (cudaFuncSetAttribute(P->g13, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)moe_gemm_smem_bytes()) != cudaSuccess ||
        cudaFuncSetAttribute(P->g2, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)moe_gemm_smem_bytes()) != cudaSuccess) {
      cudaGetLastError();
      P->gemm_ok = false;
    }
  }
  {
    auto padw = [](size_t n) { return n + n / 32; };
    const size_t budget = 74 * 1024;      // three CTAs per SM
    const size_t mid_row = 4 * (padw(std::max(d->w13_out, d->inter)) + padw(d->inter)), out_row = 4 * padw(d->hidden);
    P->mid_sg = (int)std::max<size_t>(1, std::min<size_t>(8, budget / mid_row));
    P->out_rg = (int)std::max<size_t>(1, std::min<size_t>(std::min(8, d->top_k), budget / out_row));
    // running sums between passes are only needed when one pass cannot hold all routings of a token
    const size_t out_fixed = P->out_rg < d->top_k ? 4 * (size_t)d->hidden : 0;
    P->mid_smem = P->mid_sg * mid_row;
    P->out_smem = P->out_rg * out_row + out_fixed;
    if (cudaFuncSetAttribute(moe_group_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)((4 * d->num_experts + 1) * sizeof(int))) != cudaSuccess ||
        cudaFuncSetAttribute(moe_mid_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P->mid_smem) != cudaSuccess ||
        cudaFuncSetAttribute(moe_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)P->out_smem) != cudaSuccess) {
      delete P;
      return moe_fail(GLQB_E_CUDA, "moe_plan_create: %s", cudaGetErrorString(cudaGetLastError()));
    }
  }
  if (e8 && !P->gemm_ok) {
    delete P;
    return moe_fail(GLQB_E_INVALID, "moe_plan_create: the tensor-core form is unavailable for these E8 experts");
  }
  int dev_id = 0;
  if (cudaGetDevice(&dev_id) != cudaSuccess ||
      cudaDeviceGetAttribute(&P->sm_count, cudaDevAttrMultiProcessorCount, dev_id) != cudaSuccess) {
    delete P;
    return moe_fail(GLQB_E_CUDA, "moe_plan_create: no CUDA device");
  }
  const int units13 = M.E * (d->w13_out / 32) * M.kch13, units2 = M.E * (d->hidden / 32) * M.kch2;
  const int ctas = P->sm_count * 2;
  P->grid13 = std::max(1, std::min(ctas, (units13 + MV_WARPS - 1) / MV_WARPS));
  P->grid2 = std::max(1, std::min(ctas, (units2 + MV_WARPS - 1) / MV_WARPS));
  *out = P;
  return GLQB_OK;
}

size_t glqb_moe_plan_workspace_bytes(const GlqbMoePlan* p) { return p ? p->ws_bytes : 0; }

int64_t glqb_moe_plan_code_bytes(const GlqbMoePlan* p) {
  if (!p) return 0;
  const MoeDev& M = p->dev;
  if (M.format == GLQB_FMT_E8_SHELL) return (int64_t)M.E * M.e8_ns * (M.w13_stride[0] + M.w2_stride[0]);
  return (int64_t)M.E * (M.w13_stride[0] + M.w13_stride[1] + M.w2_stride[0] + M.w2_stride[1]);
}

int glqb_moe_plan_run(GlqbMoePlan* P, const void* x, const void* topk_ids, const float* topk_weights, void* y,
                      int32_t tokens, void* workspace, size_t workspace_bytes, void* stream_) {
  if (!P || !x || !topk_ids || !topk_weights || !y) return moe_fail(GLQB_E_INVALID, "moe_plan_run: null argument");
  if (tokens < 1 || tokens > P->desc.max_tokens)
    return moe_fail(GLQB_E_INVALID, "moe_plan_run: %d tokens, plan was built for at most %d", tokens, P->desc.max_tokens);
  if (!workspace || workspace_bytes < P->ws_bytes)
    return moe_fail(GLQB_E_WORKSPACE, "moe_plan_run: workspace of %zu bytes needed, %zu given", P->ws_bytes, workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return moe_fail(GLQB_E_WORKSPACE, "workspace must be 256-byte aligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream_);
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  if (P->gemm_ok && (P->dev.format == GLQB_FMT_E8_SHELL ||
                     (long long)tokens * P->dev.top_k >= (long long)P->dev.E * moe_gemm_min_avg())) {
    const MoeDev& G = P->devg;
    const int R = tokens * G.top_k;
    moe_launch_group(G, topk_ids, tokens, ws, st);
    moe_rht_in_gemm_kernel<<<tokens, std::max(64, std::min(1024, G.hidden / 8)), G.hidden * 4, st>>>(
        G, reinterpret_cast<const uint8_t*>(x), ws);
    int* status = reinterpret_cast<int*>(ws + G.o_status);
    const int* nitems = reinterpret_cast<const int*>(ws + G.o_nitems);
    {
      MoeTimer t(P, st);
      P->g13<<<std::min(P->sm_count, G.max_items13), GM_THREADS, moe_gemm_smem_bytes(), st>>>(
          reinterpret_cast<const DevLinear*>(ws + G.o_layers13), reinterpret_cast<const GemmItem*>(ws + G.o_items13),
          G.max_items13, ws, status, nitems);
    }
    moe_mid_kernel<<<(R + P->mid_sg - 1) / P->mid_sg, MOE_XF_THREADS, P->mid_smem, st>>>(G, tokens, P->mid_sg, ws);
    {
      MoeTimer t(P, st);
      P->g2<<<std::min(P->sm_count, G.max_items2), GM_THREADS, moe_gemm_smem_bytes(), st>>>(
          reinterpret_cast<const DevLinear*>(ws + G.o_layers2), reinterpret_cast<const GemmItem*>(ws + G.o_items2),
          G.max_items2, ws, status, nitems + 1);
    }
    moe_out_kernel<<<tokens, MOE_XF_THREADS, P->out_smem, st>>>(G, tokens, P->out_rg, topk_weights, ws,
                                                               reinterpret_cast<uint8_t*>(y));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return moe_fail(GLQB_E_CUDA, "moe_plan_run: %s", cudaGetErrorString(e));
    return GLQB_OK;
  }
  const MoeDev& M = P->dev;
  const int R = tokens * M.top_k;
  moe_launch_group(M, topk_ids, tokens, ws, st);
  moe_rht_in_kernel<<<tokens, std::max(64, std::min(1024, M.hidden / 8)), M.hidden * 4, st>>>(
      M, reinterpret_cast<const uint8_t*>(x), ws);
  MoeMvArgs A;
  memset(&A, 0, sizeof A);
  A.codes[0] = M.w13[0]; A.codes[1] = M.w13[1]; A.stride[0] = M.w13_stride[0]; A.stride[1] = M.w13_stride[1];
  A.inv2 = M.w13_inv2;
  A.count = reinterpret_cast<const int*>(ws + M.o_count);
  A.base = reinterpret_cast<const int*>(ws + M.o_base);
  A.row_map = reinterpret_cast<const int*>(ws + M.o_route_tok);
  A.xr = reinterpret_cast<const __half*>(ws + M.o_xr1);
  A.part = reinterpret_cast<float*>(ws + M.o_part1);
  A.work = reinterpret_cast<int*>(ws + M.o_work);
  A.E = M.E; A.m = M.w13_out; A.n = M.hidden; A.gps = M.hidden / 32; A.strips = M.w13_out / 32;
  A.kchunks = M.kch13; A.gpc = M.gpc13; A.R = R;
  {
    MoeTimer t(P, st);
    P->k13<<<P->grid13, MV_THREADS, 0, st>>>(A);
  }
  moe_mid_kernel<<<(R + P->mid_sg - 1) / P->mid_sg, MOE_XF_THREADS, P->mid_smem, st>>>(M, tokens, P->mid_sg, ws);
  A.codes[0] = M.w2[0]; A.codes[1] = M.w2[1]; A.stride[0] = M.w2_stride[0]; A.stride[1] = M.w2_stride[1];
  A.inv2 = M.w2_inv2;
  A.row_map = nullptr;
  A.xr = reinterpret_cast<const __half*>(ws + M.o_xr2);
  A.part = reinterpret_cast<float*>(ws + M.o_part2);
  A.work = reinterpret_cast<int*>(ws + M.o_work) + 1;
  A.m = M.hidden; A.n = M.inter; A.gps = M.inter / 32; A.strips = M.hidden / 32;
  A.kchunks = M.kch2; A.gpc = M.gpc2;
  {
    MoeTimer t(P, st);
    P->k2<<<P->grid2, MV_THREADS, 0, st>>>(A);
  }
  moe_out_kernel<<<tokens, MOE_XF_THREADS, P->out_smem, st>>>(M, tokens, P->out_rg, topk_weights, ws,
                                                             reinterpret_cast<uint8_t*>(y));
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return moe_fail(GLQB_E_CUDA, "moe_plan_run: %s", cudaGetErrorString(e));
  return GLQB_OK;
}

int glqb_moe_plan_status(const GlqbMoePlan* P, const void* workspace, void* stream_) {
  if (!P || !workspace) return moe_fail(GLQB_E_INVALID, "moe_plan_status: null argument");
  if (!P->gemm_ok) return GLQB_OK;
  int st = 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  if (cudaMemcpyAsync(&st, reinterpret_cast<const uint8_t*>(workspace) + P->devg.o_status, sizeof st, cudaMemcpyDeviceToHost, s) !=
          cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess)
    return moe_fail(GLQB_E_CUDA, "moe_plan_status: %s", cudaGetErrorString(cudaGetLastError()));
  if (st != 0) return moe_fail(GLQB_E_DEVICE, "moe: a bounded wait inside the GEMM kernel gave up (role %d); results are invalid", st);
  return GLQB_OK;
}

int glqb_moe_plan_set_timing(GlqbMoePlan* P, int32_t enable) {
  if (!P) return moe_fail(GLQB_E_INVALID, "moe_plan_set_timing: null plan");
  P->timing = enable != 0;
  P->ev_used = 0;
  return GLQB_OK;
}

int glqb_moe_plan_kernel_ms(GlqbMoePlan* P, double* total_ms_out, int32_t* runs_out) {
  if (!P || !total_ms_out || !runs_out) return moe_fail(GLQB_E_INVALID, "moe_plan_kernel_ms: null argument");
  double total = 0.0;
  for (size_t i = 0; i + 1 < P->ev_used; i += 2) {
    float ms = 0.f;
    if (cudaEventSynchronize(P->ev[i + 1]) != cudaSuccess || cudaEventElapsedTime(&ms, P->ev[i], P->ev[i + 1]) != cudaSuccess)
      return moe_fail(GLQB_E_CUDA, "moe_plan_kernel_ms: %s", cudaGetErrorString(cudaGetLastError()));
    total += ms;
  }
  *total_ms_out = total;
  *runs_out = (int32_t)(P->ev_used / 4);        // two matmuls per run
  return GLQB_OK;
}

void glqb_moe_plan_destroy(GlqbMoePlan* p) {
  if (!p) return;
  for (cudaEvent_t e : p->ev) cudaEventDestroy(e);
  delete p;
}

}  // extern "C"
