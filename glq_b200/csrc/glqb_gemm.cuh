// Prefill path: decoded weight tiles -> swizzled shared memory -> tcgen05.mma with fp32 accumulators in
// tensor memory (TMEM).  One CTA computes D[128 weight rows x TN tokens] = W~[128 x K] * X~[TN x K]^T.
//
// Warp roles (GM_THREADS = 704):
//   warps 0-15 decode producers in two groups of eight; group 0 produces the even 128x64 weight chunks,
//              group 1 the odd ones (two stages are always being filled).  Inside a group every warp
//              decodes one 32x32 trellis group (or 16 rows x 64 columns of E8 indices) into the stage's
//              A tile, K-major with the 128-byte swizzle the tensor core expects
//   warps 18-21 epilogue: tcgen05.ld of the finished accumulator (two accumulators alternate, so the
//              next tile's MMAs run while these warps write the previous tile's partial sums)
//   warp  16   one thread issues tcgen05.mma (4 per chunk: K = 16 each) and tcgen05.commit
//   warp  17   one thread fetches the activation tile of the chunk with a bulk async copy (TMA, no
//              multicast); the input-transform kernel has already written the activations in the
//              exact shared-memory image (swizzled), so one contiguous copy per chunk suffices
// Stages hand over through mbarriers.  Every wait is bounded: on expiry the kernel records a status
// word, stops issuing work, frees its TMEM columns and returns.
#pragma once
#include "glqb_kernels.cuh"

namespace glqb {

constexpr int GM_THREADS = 704;
constexpr int GM_PRODUCER_WARPS = 16;     // two groups of 8
constexpr int GM_GROUP_WARPS = 8;
constexpr int GM_MMA_WARP = 16;
constexpr int GM_LOAD_WARP = 17;
constexpr int GM_EPI_WARP0 = 18;          // warps 18..21 drain the accumulators (TMEM lane quarter = warp % 4)
constexpr int GM_TILE_M = 128;
constexpr int GM_TILE_K = 64;                      // fp16 elements = 128 bytes = one swizzle row
constexpr int GM_A_BYTES = GM_TILE_M * GM_TILE_K * 2;   // 16 KiB
constexpr uint32_t GM_SPIN_LIMIT = 1u << 22;       // try_wait attempts before a wait gives up

struct GemmItem {
  int layer;       // index into the device table
  int m_tile;      // 128-row tile
  int n_tile;      // TN-token tile
  int k_begin;     // first 64-column chunk
  int k_end;       // one past the last chunk
  int slot;        // partial-sum slot this item writes
};

// ---- PTX wrappers ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
// bounded wait; false = gave up.  `abort_flag` (shared memory, optional) is set by any role of the CTA whose
// own wait ran out: the others then stop waiting at once instead of each running down its own limit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const volatile int* abort_flag = nullptr) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t it = 0; it < GM_SPIN_LIMIT; ++it) {
    uint32_t ok;
    asm volatile(
        "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
        : "=r"(ok)
        : "r"(addr), "r"(parity)
        : "memory");
    if (ok) return true;
    if (abort_flag && (it & 63u) == 63u && *abort_flag) return false;
  }
  return false;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,"
      "%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile with 128-byte swizzle: rows of 128 bytes, 8-row atoms of 1024 bytes stacked along
// M/N (stride byte offset 1024), descriptor version 1 (Blackwell), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
  d |= (uint64_t)1 << 16;                 // leading byte offset (unused for swizzled K-major) = 1
  d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset
  d |= (uint64_t)1 << 46;                 // descriptor version
  d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
  return d;
}
// instruction descriptor: D fp32, A and B fp16, both K-major, M = 128, N = tn
__device__ __forceinline__ uint32_t umma_idesc_f16(int tn) {
  return (1u << 4) | ((uint32_t)(tn >> 3) << 17) | ((uint32_t)(GM_TILE_M >> 4) << 24);
}
// byte offset of element (row r, fp16 column e) inside a swizzled K-major tile
__device__ __forceinline__ uint32_t sw128_offset(int r, int e) {
  return (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((((e >> 3) ^ (r & 7)) & 7) << 4) + (e & 7) * 2);
}

// ---- input transform for the GEMM path: activations written as swizzled TN x 64 tiles ---------------
// One CTA per (layer, Hadamard block, tile of tokens); tiles ordered [n_tile][k_chunk], each TN*128
// bytes.  Columns past n (the last chunk of a layer whose n is not a multiple of 64) are written as
// zeros by the CTAs of the last block.
static __global__ void __launch_bounds__(RHT_THREADS, GLQB_RHT_MINB) rht_in_gemm_kernel(const DevLinear* __restrict__ layers,
                                                                  const RhtItem* __restrict__ items,
                                                                  const uint8_t* __restrict__ x_base,
                                                                  uint8_t* __restrict__ ws) {
  extern __shared__ float fbuf[];
  const RhtItem it = items[blockIdx.x];
  const DevLinear& L = layers[it.layer];
  const int tn = L.gemm_tn;
  const int off = L.bn_off[it.block];
  const int logbs = L.bn_log[it.block];
  const int bs = 1 << logbs;
  const int kchunks = (L.n + GM_TILE_K - 1) / GM_TILE_K;
  const bool vec_ok = (off & 3) == 0 && act_rows_aligned4(x_base, L.x_off, L.x_stride, L.x_dtype);
  const float rs = L.x_is_rotated ? 1.0f : rsqrtf((float)bs);
  auto store1 = [&](int row, int i, float val) {
    const int token = it.tok0 + row;
    const int nt = token / tn, r = token - nt * tn;
    const int col = off + i;
    const int kc = col >> 6, e = col & 63;
    *reinterpret_cast<__half*>(ws + L.xr_off + ((size_t)nt * kchunks + kc) * tn * 128 + sw128_offset(r, e)) =
        __float2half_rn(val * rs);
  };
  auto load1 = [&](int row, int i) -> float {
    const int col = off + i;
    if (col >= L.in_f) return 0.f;
    float v = load_act(x_base, L.x_off + (long long)(it.tok0 + row) * L.x_stride + col, L.x_dtype);
    if (!L.x_is_rotated) v *= __half2float(L.sv[col]);
    return v;
  };
  if (L.x_is_rotated) {
    const int total = it.ntok << logbs;
    for (int o = threadIdx.x; o < total; o += blockDim.x) store1(o >> logbs, o & (bs - 1), load1(o >> logbs, o & (bs - 1)));
  } else {
    auto load32 = [&](int row, int i0, float (&v)[32]) { rht_load_x32(L, x_base, it.tok0 + row, off + i0, vec_ok, v); };
    uint8_t* xr = ws + L.xr_off;
    const int tok0 = it.tok0;
    // 8 consecutive columns are one 16-byte unit of a swizzled 128-byte row
    auto store8 = [&](int row, int i0, const float (&v)[8], int count) {
      const int col0 = off + i0;
      if (count == 8 && (col0 & 7) == 0) {
        const int token = tok0 + row;
        const int nt = token / tn, r = token - nt * tn;
        const __half2 a = __floats2half2_rn(v[0] * rs, v[1] * rs), b = __floats2half2_rn(v[2] * rs, v[3] * rs);
        const __half2 c = __floats2half2_rn(v[4] * rs, v[5] * rs), d = __floats2half2_rn(v[6] * rs, v[7] * rs);
        *reinterpret_cast<uint4*>(xr + ((size_t)nt * kchunks + (col0 >> 6)) * tn * 128 + sw128_offset(r, col0 & 63)) =
            make_uint4(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b),
                       *reinterpret_cast<const uint32_t*>(&c), *reinterpret_cast<const uint32_t*>(&d));
      } else {
        for (int k = 0; k < count; ++k) store1(row, i0 + k, v[k]);
      }
    };
    fht_tile8(fbuf, logbs, it.ntok, load32, load1, store8);
  }
  if (it.block == L.nbn - 1) {
    const int padc = kchunks * GM_TILE_K - L.n;
    for (int o = threadIdx.x; o < it.ntok * padc; o += blockDim.x) {
      const int tk = o / padc, col = L.n + (o - tk * padc);
      const int token = it.tok0 + tk;
      const int nt = token / tn, r = token - nt * tn;
      const int kc = col >> 6, e = col & 63;
      *reinterpret_cast<__half*>(ws + L.xr_off + ((size_t)nt * kchunks + kc) * tn * 128 + sw128_offset(r, e)) =
          __float2half_rn(0.f);
    }
  }
}

// ---- weight producers ------------------------------------------------------------------------------
// One trellis group (32 rows x 32 columns) -> its place in the 128 x 64 A tile.
__device__ __forceinline__ void st_shared_u32(uint32_t addr, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Byte offsets (inside a swizzled 128 x 64 tile) of the 16 register pairs a lane stores per group:
// entry q*4 + p with q = ni*2 + mi the 16x16 tile and p = c*2 + a the pair; fixed per thread.
__device__ __forceinline__ void gemm_lane_offsets(int strip, int cg, int lane, uint32_t (&off)[16]) {
  const int g = lane >> 2, t = lane & 3;
#pragma unroll
  for (int q = 0; q < 4; ++q)
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const int ni = q >> 1, mi = q & 1, c = p >> 1, a_ = p & 1;
      off[q * 4 + p] = sw128_offset(strip * 32 + mi * 16 + 8 * a_ + g, cg * 32 + ni * 16 + 8 * c + 2 * t);
    }
}

template <int K1, int K2>
__device__ __forceinline__ void gemm_store_group(uint32_t a_tile, const uint32_t (&off)[16], int lane, const Words<K1>& v,
                                                 const Words<(K2 > 0 ? K2 : 1)>& v2, __half2 s2) {
  const Words<K1> vn = shfl_words<K1>(v, (lane + 1) & 31);
  Words<K1> vn2 = vn;
  if constexpr (K1 == 1) vn2 = shfl_words<K1>(v, (lane + 2) & 31);
  Words<(K2 > 0 ? K2 : 1)> un, un2;
  if constexpr (K2 > 0) {
    un = shfl_words<K2>(v2, (lane + 1) & 31);
    un2 = un;
    if constexpr (K2 == 1) un2 = shfl_words<K2>(v2, (lane + 2) & 31);
  }
#pragma unroll
  for (int ni = 0; ni < 2; ++ni) {
#pragma unroll
    for (int mi = 0; mi < 2; ++mi) {
      const int q = ni * 2 + mi;
      uint32_t a[8], b[8];
      decode_tile<K1>(chunk_of<K1>(v, q), chunk_of<K1>(vn, q), chunk_of<K1>(vn2, q), a);
      if constexpr (K2 > 0) decode_tile<K2>(chunk_of<K2>(v2, q), chunk_of<K2>(un, q), chunk_of<K2>(un2, q), b);
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        uint32_t w = __byte_perm(a[2 * p], a[2 * p + 1], 0x5410);        // (w_{2p}, w_{2p+1})
        if constexpr (K2 > 0) {
          // second stage folded into the fp16 operand: w = fp16(w1 + s2 * w2), one rounding
          const uint32_t w2 = __byte_perm(b[2 * p], b[2 * p + 1], 0x5410);
          const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&w2), s2, *reinterpret_cast<const __half2*>(&w));
          w = *reinterpret_cast<const uint32_t*>(&r);
        }
        st_shared_u32(a_tile + off[q * 4 + p], w);
      }
    }
  }
}

// ---- the GEMM kernel -------------------------------------------------------------------------------
// FORMAT 0: trellis (K1, K2 bits); FORMAT 1: E8 (K1 = number of stages, K2 unused);
// FORMAT 2: the weight tiles were decoded beforehand (e8_tiles_kernel) and are fetched like the
//           activation tiles, one bulk copy per stage; the producer warps have nothing to do
template <int FORMAT, int K1, int K2, int TN, int STAGES>
__global__ void __launch_bounds__(GM_THREADS, 1)
glq_gemm_kernel(const DevLinear* __restrict__ layers, const GemmItem* __restrict__ items, int n_items,
                uint8_t* __restrict__ ws, int* __restrict__ status, const int* __restrict__ n_items_dev) {
  // work lists built on the device (grouped expert matmul) pass their length through memory
  if (n_items_dev) n_items = min(n_items, *n_items_dev);
  constexpr int B_BYTES = TN * 128;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* a_base = smem;                                   // STAGES x 16 KiB
  uint8_t* b_base = smem + STAGES * GM_A_BYTES;             // STAGES x TN*128
  uint64_t* bars = reinterpret_cast<uint64_t*>(b_base + STAGES * B_BYTES);
  uint64_t* full_a = bars;
  uint64_t* full_b = bars + STAGES;
  uint64_t* empty = bars + 2 * STAGES;
  uint64_t* acc_full = bars + 3 * STAGES;          // [2]
  uint64_t* acc_empty = acc_full + 2;              // [2]
  uint64_t* drain = acc_empty + 2;                 // give-up path only: completion of the MMAs issued so far
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(drain + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_a[s], GM_GROUP_WARPS);
      mbar_init(&full_b[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
    }
    mbar_init(drain, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == GM_MMA_WARP) {
    tmem_alloc(tmem_slot, 2 * TN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_acc = *tmem_slot;
  uint32_t loads_issued = 0;                       // activation-loader thread: stages armed so far

  if (warp < GM_PRODUCER_WARPS) {
    // ------------------------------------------------------------------ producers (+ epilogue)
    // q numbers the chunks of this CTA over all its items; chunk q lives in stage q % STAGES and is
    // produced by group (q & 1).  Every role derives stage and phase from q in the same way.
    const int grp = warp >> 3, wl = warp & 7;
    uint32_t q0 = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
      const GemmItem it = items[item];
      const DevLinear& L = layers[it.layer];
      const int first = it.k_begin + (int)((grp - q0) & 1u);       // this group's first chunk of the item
      if constexpr (FORMAT == 2) {
        (void)first; (void)wl; (void)L;
      } else if constexpr (FORMAT == 0) {
        const int strip = wl >> 1, cg = wl & 1;
        const int rp = it.m_tile * 4 + strip;
        const int gps = L.groups_per_strip;
        const bool row_ok = rp < L.strips;
        const uint8_t* p1 = L.codes[0] + ((long long)rp * gps) * (128 * K1) + lane * (4 * K1);
        const uint8_t* p2 = nullptr;
        if constexpr (K2 > 0) p2 = L.codes[1] + ((long long)rp * gps) * (128 * K2) + lane * (4 * K2);
        const __half2 s2 = __float2half2_rn(L.stage_scale[1]);
        uint32_t off[16];
        gemm_lane_offsets(strip, cg, lane, off);
        Words<K1> nxt;
        Words<(K2 > 0 ? K2 : 1)> nxt2;
        auto fetch = [&](int kc) {
          const int cp = kc * 2 + cg;
          if (row_ok && cp < gps) {
            nxt = load_words<K1>(p1 + (long long)cp * (128 * K1));
            if constexpr (K2 > 0) nxt2 = load_words<K2>(p2 + (long long)cp * (128 * K2));
          }
        };
        if (first < it.k_end) fetch(first);
        for (int kc = first; kc < it.k_end; kc += 2) {
          const uint32_t q = q0 + (uint32_t)(kc - it.k_begin);
          const int stage = (int)(q % STAGES);
          const uint32_t phase = (q / STAGES) & 1u;
          const Words<K1> v = nxt;
          const Words<(K2 > 0 ? K2 : 1)> v2 = nxt2;
          const bool valid = row_ok && (kc * 2 + cg) < gps;
          if (kc + 2 < it.k_end) fetch(kc + 2);
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t a_tile = smem_u32(a_base) + stage * GM_A_BYTES;
          if (valid) {
            gemm_store_group<K1, K2>(a_tile, off, lane, v, v2, s2);
          } else {
            // rows or columns past the matrix: zeros (validity is uniform per warp, so the shuffles
            // inside the decode always see all 32 lanes)
#pragma unroll
            for (int i = 0; i < 16; ++i) st_shared_u32(a_tile + off[i], 0u);
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full_a[stage]);
        }
      } else {
        // E8: 128 rows x 8 indices per chunk; thread (row = tid >> 1, half = tid & 1) expands 4 indices
        const int tid = threadIdx.x & 255;                // thread inside the producer group
        const int row_l = tid >> 1, hf = tid & 1;
        const int row = it.m_tile * GM_TILE_M + row_l;
        const int nidx = L.n >> 3;
        const bool row_ok = row < L.m;
        // 8-byte loads need every row (and the matrix itself) to start on an 8-byte boundary
        bool vec_ok = (nidx & 3) == 0;
#pragma unroll
        for (int s = 0; s < K1; ++s) vec_ok = vec_ok && (reinterpret_cast<uintptr_t>(L.codes[s]) & 7) == 0;
        uint2 nq[K1];                                     // 4 indices (8 bytes) per stage
        auto fetch = [&](int kc) {
          const int i0 = kc * 8 + hf * 4;
#pragma unroll
          for (int s = 0; s < K1; ++s) {
            nq[s] = make_uint2(0u, 0u);
            if (row_ok && vec_ok && i0 + 4 <= nidx) {
              nq[s] = ld_stream_v2(reinterpret_cast<const uint16_t*>(L.codes[s]) + (long long)row * nidx + i0);
            } else if (row_ok) {
              const uint16_t* qd = reinterpret_cast<const uint16_t*>(L.codes[s]) + (long long)row * nidx;
              uint32_t v[4] = {0, 0, 0, 0};
              for (int k = 0; k < 4; ++k) if (i0 + k < nidx) v[k] = qd[i0 + k];
              nq[s] = make_uint2(v[0] | (v[1] << 16), v[2] | (v[3] << 16));
            }
          }
        };
        if (first < it.k_end) fetch(first);
        for (int kc = first; kc < it.k_end; kc += 2) {
          const uint32_t q = q0 + (uint32_t)(kc - it.k_begin);
          const int stage = (int)(q % STAGES);
          const uint32_t phase = (q / STAGES) & 1u;
          uint2 cq[K1];
#pragma unroll
          for (int s = 0; s < K1; ++s) cq[s] = nq[s];
          if (kc + 2 < it.k_end) fetch(kc + 2);
          // gather before waiting for the stage: the table reads overlap the wait
          uint32_t ent[K1][4];
          const int i0 = kc * 8 + hf * 4;
#pragma unroll
          for (int s = 0; s < K1; ++s) {
            const uint32_t mask = (uint32_t)L.table_entries[s] - 1u;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint32_t idx = ((k < 2 ? cq[s].x : cq[s].y) >> ((k & 1) * 16)) & 0xFFFFu;
              ent[s][k] = __ldg(L.table[s] + (idx & mask));
            }
          }
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          const uint32_t a_tile = smem_u32(a_base) + stage * GM_A_BYTES;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint4 out = make_uint4(0u, 0u, 0u, 0u);
            if (row_ok && i0 + k < nidx) {
              uint32_t h[4];
              e8_entry_to_half2(ent[0][k], h);               // (c0,c4),(c1,c5),(c2,c6),(c3,c7)
#pragma unroll
              for (int s = 1; s < K1; ++s) {
                uint32_t h2[4];
                e8_entry_to_half2(ent[s][k], h2);
                const __half2 sc = __float2half2_rn(L.stage_scale[s]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&h2[j]), sc,
                                            *reinterpret_cast<const __half2*>(&h[j]));
                  h[j] = *reinterpret_cast<const uint32_t*>(&r);
                }
              }
              // natural column order inside the 16-byte chunk: (c0,c1),(c2,c3),(c4,c5),(c6,c7)
              out.x = __byte_perm(h[0], h[1], 0x5410);
              out.y = __byte_perm(h[2], h[3], 0x5410);
              out.z = __byte_perm(h[0], h[1], 0x7632);
              out.w = __byte_perm(h[2], h[3], 0x7632);
            }
            st_shared_v4(a_tile + sw128_offset(row_l, (hf * 4 + k) * 8), out);
          }
          fence_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&full_a[stage]);
        }
      }
      q0 += (uint32_t)(it.k_end - it.k_begin);
      if (!ok) break;
    }
    if (!ok) { *abort_flag = 1; if (lane == 0) atomicCAS(status, 0, (int)ST_GAVE_UP_PRODUCER); }
  } else if (warp == GM_MMA_WARP) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, seq = 0;
      const uint32_t idesc = umma_idesc_f16(TN);
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++seq) {
        const GemmItem it = items[item];
        const uint32_t a = seq & 1u, a_phase = (seq >> 1) & 1u;     // accumulator and its use count parity
        const uint32_t d_tmem = tmem_acc + a * TN;
        if (!mbar_wait(&acc_empty[a], a_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        for (int kc = it.k_begin; kc < it.k_end; ++kc) {
          if ((FORMAT != 2 && !mbar_wait(&full_a[stage], phase, abort_flag)) || !mbar_wait(&full_b[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint64_t da = umma_desc_sw128(smem_u32(a_base + stage * GM_A_BYTES));
          const uint64_t db = umma_desc_sw128(smem_u32(b_base + stage * B_BYTES));
#pragma unroll
          for (int k = 0; k < GM_TILE_K / 16; ++k)      // +32 bytes (2 x 16-byte units) per K step of 16
            umma_f16(d_tmem, da + (uint64_t)(2 * k), db + (uint64_t)(2 * k), idesc, (kc > it.k_begin || k > 0) ? 1u : 0u);
          umma_commit(&empty[stage]);                    // stage reusable once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&acc_full[a]);
      }
      if (!ok) { *abort_flag = 1; atomicCAS(status, 0, (int)ST_GAVE_UP_MMA); }
    }
  } else if (warp == GM_LOAD_WARP) {
    // ------------------------------------------------------------------ activation loader
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
        const GemmItem it = items[item];
        const DevLinear& L = layers[it.layer];
        const int kchunks = (L.n + GM_TILE_K - 1) / GM_TILE_K;
        const uint8_t* src = ws + L.xr_off + ((size_t)it.n_tile * kchunks) * B_BYTES;
        for (int kc = it.k_begin; kc < it.k_end; ++kc) {
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          if constexpr (FORMAT == 2) {
            mbar_expect_tx(&full_b[stage], B_BYTES + GM_A_BYTES);
            bulk_g2s(a_base + stage * GM_A_BYTES,
                     ws + L.atile_off + ((size_t)it.m_tile * kchunks + kc) * GM_A_BYTES, GM_A_BYTES, &full_b[stage]);
          } else {
            mbar_expect_tx(&full_b[stage], B_BYTES);
          }
          bulk_g2s(b_base + stage * B_BYTES, src + (size_t)kc * B_BYTES, B_BYTES, &full_b[stage]);
          ++loads_issued;
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
      if (!ok) { *abort_flag = 1; atomicCAS(status, 0, (int)ST_GAVE_UP_LOADER); }
    }
  }
  else {
    // ------------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;                          // TMEM lanes 32*quarter .. 32*quarter + 31
    uint32_t seq = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ++seq) {
      const GemmItem it = items[item];
      const DevLinear& L = layers[it.layer];
      const uint32_t a = seq & 1u, a_phase = (seq >> 1) & 1u;
      if (!mbar_wait(&acc_full[a], a_phase, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int row = it.m_tile * GM_TILE_M + quarter * 32 + lane;
      float* part = reinterpret_cast<float*>(ws + L.part_off) + (long long)it.slot * L.batch * L.m;
#pragma unroll 1
      for (int c0 = 0; c0 < TN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_acc + ((uint32_t)(quarter * 32) << 16) + a * TN + (uint32_t)c0, r);
        tmem_ld_wait();
        if (row < L.m) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int token = it.n_tile * TN + c0 + i;
            if (token < L.batch) part[(long long)token * L.m + row] = __uint_as_float(r[i]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[a]);
    }
    if (!ok) { *abort_flag = 1; if (lane == 0) atomicCAS(status, 0, (int)ST_GAVE_UP_EPILOGUE); }
  }
  // ---- teardown: every thread arrives here (also after a wait gave up)
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A role gave up.  Before shared memory and tensor memory are released, wait (bounded again) for what
    // may still be in flight: the bulk copies into the stages armed last, and the MMAs issued so far.
    if (warp == GM_LOAD_WARP && lane == 0) {
      const uint32_t n = loads_issued < (uint32_t)STAGES ? loads_issued : (uint32_t)STAGES;
      for (uint32_t i = 0; i < n; ++i) {
        const uint32_t q = loads_issued - 1 - i;
        mbar_wait(&full_b[q % STAGES], (q / STAGES) & 1u);
      }
    }
    if (warp == GM_MMA_WARP && lane == 0) {
      umma_commit(drain);
      mbar_wait(drain, 0);
    }
    tc_fence_before();
    __syncthreads();
  }
  if (warp == GM_MMA_WARP) tmem_dealloc(tmem_acc, 2 * TN);
}

// ---- decode once: E8 indices -> swizzled fp16 weight tiles in global memory ----------------------------
// For large token counts the fused kernel would decode every weight tile once per token tile; this
// kernel decodes each 128 x 64 tile ONCE into the exact shared-memory image (K-major, 128-byte swizzle),
// [m_tile][k_chunk] x 16 KiB, which glq_gemm_kernel<2,...> then fetches with one bulk copy per stage.
// A CTA takes 128 rows x 4 consecutive chunks; thread (row = tid >> 1, half = tid & 1) reads the 16 indices
// of two chunks with two 16-byte loads per stage (the two threads of a row read 64 contiguous bytes), keeps
// all 16 * NS gathers in flight, and writes two full 128-byte tile rows.
// TM = 0: table gathers from global memory, one unit per 256-thread CTA.  TM = 1: most of the table resident in
// shared memory (see e8_gather), 512-thread CTA = two units side by side, one CTA per SM.
template <int NS, int TM>
__device__ __forceinline__ void e8_tiles_body(const DevLinear* __restrict__ layers, int first, int count,
                                              uint8_t* __restrict__ ws, const E8Tables& T, int unit0, int unit_stride,
                                              int tid) {
  const int row_l = tid >> 1, hf = tid & 1;
  for (int li = first; li < first + count; ++li) {
    const DevLinear& L = layers[li];
    const int kchunks = (L.n + GM_TILE_K - 1) / GM_TILE_K;
    const int m_tiles = (L.m + GM_TILE_M - 1) / GM_TILE_M;
    const int kgroups = (kchunks + 3) >> 2;
    const int nidx = L.n >> 3, m = L.m;
    bool vec_ok = (nidx & 7) == 0;                       // every row starts 16-byte aligned
    const uint16_t* codes[NS];
    E8Stage stg[NS];
    __half2 sc[NS];
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      codes[s] = reinterpret_cast<const uint16_t*>(L.codes[s]);
      vec_ok = vec_ok && (reinterpret_cast<uintptr_t>(L.codes[s]) & 15) == 0;
      stg[s].table = L.table[s];
      stg[s].mask = (uint32_t)L.table_entries[s] - 1u;
      stg[s].base = L.table_entries[s] == 65536 ? T.table_base : T.small_base;
      sc[s] = __float2half2_rn(L.stage_scale[s]);
    }
    uint8_t* tiles = ws + L.atile_off;
    for (int u = unit0; u < m_tiles * kgroups; u += unit_stride) {
      const int mt = u / kgroups, kg = u - mt * kgroups;
      const int row = mt * GM_TILE_M + row_l;
      const bool row_ok = row < m;
      const int kc0 = kg * 4 + hf * 2;
      uint32_t ent[NS][2][8];
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        const uint16_t* q = codes[s] + (long long)row * nidx;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int i0 = (kc0 + c) * 8;
          uint32_t w[4] = {0u, 0u, 0u, 0u};
          if (row_ok && vec_ok && i0 + 8 <= nidx) {
            const uint4 t = ld_stream_v4(q + i0);
            w[0] = t.x; w[1] = t.y; w[2] = t.z; w[3] = t.w;
          } else if (row_ok) {
#pragma unroll
            for (int k = 0; k < 8; ++k)
              if (i0 + k < nidx) w[k >> 1] |= (uint32_t)q[i0 + k] << ((k & 1) * 16);
          }
#pragma unroll
          for (int k = 0; k < 8; ++k)
            ent[s][c][k] = e8_gather<TM>(stg[s], ((w[k >> 1] >> ((k & 1) * 16)) & 0xFFFFu) & stg[s].mask);
        }
      }
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int kc = kc0 + c;
        if (kc >= kchunks) continue;
        uint8_t* tile = tiles + ((size_t)mt * kchunks + kc) * GM_A_BYTES;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          uint4 out = make_uint4(0u, 0u, 0u, 0u);
          if (row_ok && kc * 8 + k < nidx) {
            uint32_t h[4];
            e8_entry_to_half2(ent[0][c][k], h);
#pragma unroll
            for (int s = 1; s < NS; ++s) {
              uint32_t h2[4];
              e8_entry_to_half2(ent[s][c][k], h2);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&h2[j]), sc[s], *reinterpret_cast<const __half2*>(&h[j]));
                h[j] = *reinterpret_cast<const uint32_t*>(&r);
              }
            }
            // natural column order inside the 16-byte chunk: (c0,c1),(c2,c3),(c4,c5),(c6,c7)
            out.x = __byte_perm(h[0], h[1], 0x5410);
            out.y = __byte_perm(h[2], h[3], 0x5410);
            out.z = __byte_perm(h[0], h[1], 0x7632);
            out.w = __byte_perm(h[2], h[3], 0x7632);
          }
          *reinterpret_cast<uint4*>(tile + sw128_offset(row_l, k * 8)) = out;
        }
      }
    }
  }
}

template <int NS>
__global__ void __launch_bounds__(256) e8_tiles_kernel(const DevLinear* __restrict__ layers, int first, int count,
                                                       uint8_t* __restrict__ ws) {
  const E8Tables T = {0u, 0u};
  e8_tiles_body<NS, 0>(layers, first, count, ws, T, blockIdx.x, gridDim.x, threadIdx.x);
}

constexpr int E8TS_THREADS = 512;
template <int NS>
__global__ void __launch_bounds__(E8TS_THREADS, 1)
e8_tiles_smem_kernel(const DevLinear* __restrict__ layers, int first, int count, uint8_t* __restrict__ ws,
                     const uint32_t* __restrict__ big_table, const uint32_t* __restrict__ small_table, int small_entries) {
  extern __shared__ __align__(16) uint32_t e8t_smem[];
  const uint4* src = reinterpret_cast<const uint4*>(big_table);
  uint4* dst = reinterpret_cast<uint4*>(e8t_smem);
  for (int i = threadIdx.x; i < E8S_RESIDENT / 4; i += blockDim.x) dst[i] = __ldg(src + i);
  for (int i = threadIdx.x; i < small_entries && i < 256; i += blockDim.x) e8t_smem[E8S_RESIDENT + i] = __ldg(small_table + i);
  E8Tables T;
  const uint32_t local = (uint32_t)__cvta_generic_to_shared(e8t_smem);
  T.table_base = local;
  T.small_base = local + E8S_RESIDENT * 4;
  __syncthreads();
  e8_tiles_body<NS, 1>(layers, first, count, ws, T, blockIdx.x * 2 + (threadIdx.x >> 8), gridDim.x * 2, threadIdx.x & 255);
}

}  // namespace glqb
