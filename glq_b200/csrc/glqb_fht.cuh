// In-CTA Walsh-Hadamard transform on a shared-memory buffer.
// Butterfly order follows the reference (glq/hadamard.py:18-26, glq/csrc/glq_fht.cuh:14-21):
// stages in ascending distance 1,2,4,...; the lower index of a pair receives a+b, the upper a-b.
// The caller applies the 1/sqrt(bs) normalisation.
#pragma once
#include "glqb_internal.h"

namespace glqb {

template <int R>   // R = number of stages done in registers this pass (1..3)
__device__ __forceinline__ void fht_pass(float* buf, int bs, int done) {
  constexpr int N = 1 << R;
  const int stride = 1 << done;
  const int ngroups = bs >> R;
  for (int o = threadIdx.x; o < ngroups; o += blockDim.x) {
    const int low = o & (stride - 1);
    const int high = o >> done;
    const int base = (high << (done + R)) | low;
    float v[N];
#pragma unroll
    for (int k = 0; k < N; ++k) v[k] = buf[base + k * stride];
#pragma unroll
    for (int s = 0; s < R; ++s) {
#pragma unroll
      for (int k = 0; k < N; ++k) {
        if (!(k & (1 << s))) {
          float a = v[k], b = v[k | (1 << s)];
          v[k] = a + b;
          v[k | (1 << s)] = a - b;
        }
      }
    }
#pragma unroll
    for (int k = 0; k < N; ++k) buf[base + k * stride] = v[k];
  }
}

// All threads of the CTA must call this; buf holds bs = 2^logbs floats and is fully written.
__device__ __forceinline__ void fht_smem(float* buf, int logbs) {
  const int bs = 1 << logbs;
  int done = 0;
  __syncthreads();
  while (done < logbs) {
    const int r = min(3, logbs - done);
    if (r == 3) fht_pass<3>(buf, bs, done);
    else if (r == 2) fht_pass<2>(buf, bs, done);
    else fht_pass<1>(buf, bs, done);
    __syncthreads();
    done += r;
  }
}

// Several rows at once: buf holds `rows` consecutive arrays of 2^logbs floats; each row is transformed
// independently.  The (row, butterfly group) pairs are spread over all threads, so a CTA that owns a
// tile of tokens of a small Hadamard block keeps every thread busy.
template <int R>
__device__ __forceinline__ void fht_pass_rows(float* buf, int logbs, int done, int rows) {
  constexpr int N = 1 << R;
  const int stride = 1 << done;
  const int glog = logbs - R;                 // log2(groups per row)
  const int total = rows << glog;
  for (int o = threadIdx.x; o < total; o += blockDim.x) {
    const int row = o >> glog;
    const int oo = o & ((1 << glog) - 1);
    const int low = oo & (stride - 1);
    const int high = oo >> done;
    float* p = buf + ((size_t)row << logbs) + ((high << (done + R)) | low);
    float v[N];
#pragma unroll
    for (int k = 0; k < N; ++k) v[k] = p[k * stride];
#pragma unroll
    for (int s = 0; s < R; ++s) {
#pragma unroll
      for (int k = 0; k < N; ++k) {
        if (!(k & (1 << s))) {
          float a = v[k], b = v[k | (1 << s)];
          v[k] = a + b;
          v[k | (1 << s)] = a - b;
        }
      }
    }
#pragma unroll
    for (int k = 0; k < N; ++k) p[k * stride] = v[k];
  }
}

__device__ __forceinline__ void fht_smem_rows(float* buf, int logbs, int rows) {
  int done = 0;
  __syncthreads();
  while (done < logbs) {
    const int r = min(3, logbs - done);
    if (r == 3) fht_pass_rows<3>(buf, logbs, done, rows);
    else if (r == 2) fht_pass_rows<2>(buf, logbs, done, rows);
    else fht_pass_rows<1>(buf, logbs, done, rows);
    __syncthreads();
    done += r;
  }
}

}  // namespace glqb

// ---------------------------------------------------------------------------------------------------
// Tiled transform with radix-32 register passes.
//
// A tile is `rows` independent arrays of 2^logbs values.  Pass 1 is fused with the load: a thread pulls
// 32 consecutive values straight from global memory (the caller's `load32`), does butterfly stages 0-4 in
// registers and parks them in shared memory; the last pass is fused with the store (`store1` receives
// every finished value).  Arrays of up to 32 values never touch shared memory, up to 1024 values make one
// round trip, up to 32768 two.  Shared memory is padded by one word per 32 (index i lives at i + i/32), which
// makes the 32-consecutive accesses of pass 1 and the strided accesses of the later passes conflict-free.
// Butterfly order is the reference's: ascending distance, lower index gets a+b.
// ---------------------------------------------------------------------------------------------------
namespace glqb {

__device__ __forceinline__ int fht_pad(int i) { return i + (i >> 5); }
__host__ __device__ __forceinline__ int fht_tile_words(int logbs, int rows) {
  const int bs = 1 << logbs;
  return rows * (bs + (bs >> 5));
}

template <int R>
__device__ __forceinline__ void fht_regs(float (&v)[1 << R]) {
#pragma unroll
  for (int s = 0; s < R; ++s) {
#pragma unroll
    for (int k = 0; k < (1 << R); ++k) {
      if (!(k & (1 << s))) {
        const float a = v[k], b = v[k | (1 << s)];
        v[k] = a + b;
        v[k | (1 << s)] = a - b;
      }
    }
  }
}

// last pass: R remaining stages at distance 2^done; every finished value goes to store1(row, index, value)
template <int R, class Store1>
__device__ __forceinline__ void fht_last_pass(const float* smem, int logbs, int done, int rows, int row_words,
                                              Store1& store1) {
  const int S = 1 << done;                     // R == logbs - done: one group spans the whole array
  const int total = rows << done;
  for (int o = threadIdx.x; o < total; o += blockDim.x) {
    const int row = o >> done, low = o & (S - 1);
    const float* p = smem + row * row_words;
    float v[1 << R];
#pragma unroll
    for (int k = 0; k < (1 << R); ++k) v[k] = p[fht_pad(low + k * S)];
    fht_regs<R>(v);
#pragma unroll
    for (int k = 0; k < (1 << R); ++k) store1(row, low + k * S, v[k]);
  }
}

template <class Load32, class Load1, class Store1>
__device__ __forceinline__ void fht_tile(float* smem, int logbs, int rows, Load32 load32, Load1 load1, Store1 store1) {
  const int bs = 1 << logbs;
  if (logbs < 5) {
    // tiny arrays (E8 layers whose width is not a multiple of 32): one thread per array, all in registers
    for (int row = threadIdx.x; row < rows; row += blockDim.x) {
      float v[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) v[k] = k < bs ? load1(row, k) : 0.f;
      for (int h = 1; h < bs; h <<= 1)
#pragma unroll
        for (int k = 0; k < 16; ++k)
          if (!(k & h) && (k | h) < bs) { const float a = v[k], b = v[k | h]; v[k] = a + b; v[k | h] = a - b; }
#pragma unroll
      for (int k = 0; k < 16; ++k) if (k < bs) store1(row, k, v[k]);
    }
    return;
  }
  const int row_words = bs + (bs >> 5);
  const int slog = logbs - 5;                  // log2(32-value segments per array)
  const int nseg = rows << slog;
  for (int s = threadIdx.x; s < nseg; s += blockDim.x) {
    const int row = s >> slog, i0 = (s & ((1 << slog) - 1)) << 5;
    float v[32];
    load32(row, i0, v);
    fht_regs<5>(v);
    if (logbs == 5) {
#pragma unroll
      for (int k = 0; k < 32; ++k) store1(row, k, v[k]);
    } else {
      float* p = smem + row * row_words + fht_pad(i0);
#pragma unroll
      for (int k = 0; k < 32; ++k) p[k] = v[k];
    }
  }
  if (logbs == 5) return;
  __syncthreads();
  int done = 5;
  if (logbs > 10) {
    // middle pass: stages 5..9 (distance 32..512), in place
    const int total = rows << slog;
    for (int o = threadIdx.x; o < total; o += blockDim.x) {
      const int row = o >> slog, oo = o & ((1 << slog) - 1);
      const int low = oo & 31, high = oo >> 5;
      float* p = smem + row * row_words;
      const int base = (high << 10) | low;
      float v[32];
#pragma unroll
      for (int k = 0; k < 32; ++k) v[k] = p[fht_pad(base + (k << 5))];
      fht_regs<5>(v);
#pragma unroll
      for (int k = 0; k < 32; ++k) p[fht_pad(base + (k << 5))] = v[k];
    }
    __syncthreads();
    done = 10;
  }
  switch (logbs - done) {
    case 1: fht_last_pass<1>(smem, logbs, done, rows, row_words, store1); break;
    case 2: fht_last_pass<2>(smem, logbs, done, rows, row_words, store1); break;
    case 3: fht_last_pass<3>(smem, logbs, done, rows, row_words, store1); break;
    case 4: fht_last_pass<4>(smem, logbs, done, rows, row_words, store1); break;
    default: fht_last_pass<5>(smem, logbs, done, rows, row_words, store1); break;
  }
}

// ---------------------------------------------------------------------------------------------------
// Same transform with vector output: after the last butterfly pass the finished values go back to shared
// memory and every thread hands 8 consecutive values of one array to `store8(row, i0, v, count)` (count < 8
// only for arrays shorter than 8), so the caller can scale, convert and store them with one 16-byte access.
// The stages after the first five are split evenly over one or two strided in-place passes
// (2048 values: 5 + 3 + 3, 8192: 5 + 4 + 4), which keeps every pass at 8 or more values per thread.
// ---------------------------------------------------------------------------------------------------
template <int R>
__device__ __forceinline__ void fht_strided_pass(float* smem, int logbs, int done, int rows, int row_words) {
  const int S = 1 << done;
  const int glog = logbs - R;
  const int total = rows << glog;
  for (int o = threadIdx.x; o < total; o += blockDim.x) {
    const int row = o >> glog, oo = o & ((1 << glog) - 1);
    const int low = oo & (S - 1), high = oo >> done;
    float* p = smem + row * row_words + fht_pad(((high << (done + R)) | low));
    const int step = S + (S >> 5);             // S is a multiple of 32: the padding grows linearly with k
    float v[1 << R];
#pragma unroll
    for (int k = 0; k < (1 << R); ++k) v[k] = p[k * step];
    fht_regs<R>(v);
#pragma unroll
    for (int k = 0; k < (1 << R); ++k) p[k * step] = v[k];
  }
}

__device__ __forceinline__ void fht_strided_dispatch(float* smem, int logbs, int done, int r, int rows, int row_words) {
  switch (r) {
    case 1: fht_strided_pass<1>(smem, logbs, done, rows, row_words); break;
    case 2: fht_strided_pass<2>(smem, logbs, done, rows, row_words); break;
    case 3: fht_strided_pass<3>(smem, logbs, done, rows, row_words); break;
    case 4: fht_strided_pass<4>(smem, logbs, done, rows, row_words); break;
    default: fht_strided_pass<5>(smem, logbs, done, rows, row_words); break;
  }
}

// The passes alone, for arrays of 32 values or more: on return (after a __syncthreads) value i of array `row`
// sits at smem[row * (bs + bs / 32) + fht_pad(i)].
template <class Load32>
__device__ __forceinline__ void fht_tile_core(float* smem, int logbs, int rows, Load32 load32) {
  const int bs = 1 << logbs;
  const int row_words = bs + (bs >> 5);
  const int slog = logbs - 5;
  const int nseg = rows << slog;
  for (int s = threadIdx.x; s < nseg; s += blockDim.x) {
    const int row = s >> slog, i0 = (s & ((1 << slog) - 1)) << 5;
    float v[32];
    load32(row, i0, v);
    fht_regs<5>(v);
    float* p = smem + row * row_words + fht_pad(i0);
#pragma unroll
    for (int k = 0; k < 32; ++k) p[k] = v[k];
  }
  __syncthreads();
  const int rem = logbs - 5;
  if (rem > 0) {
    const int r1 = rem <= 5 ? rem : (rem + 1) >> 1;
    fht_strided_dispatch(smem, logbs, 5, r1, rows, row_words);
    __syncthreads();
    if (rem > r1) {
      fht_strided_dispatch(smem, logbs, 5 + r1, rem - r1, rows, row_words);
      __syncthreads();
    }
  }
}

template <class Load32, class Load1, class Store8>
__device__ __forceinline__ void fht_tile8(float* smem, int logbs, int rows, Load32 load32, Load1 load1, Store8 store8) {
  const int bs = 1 << logbs;
  if (logbs < 5) {
    for (int row = threadIdx.x; row < rows; row += blockDim.x) {
      float v[16];
#pragma unroll
      for (int k = 0; k < 16; ++k) v[k] = k < bs ? load1(row, k) : 0.f;
      for (int h = 1; h < bs; h <<= 1)
#pragma unroll
        for (int k = 0; k < 16; ++k)
          if (!(k & h) && (k | h) < bs) { const float a = v[k], b = v[k | h]; v[k] = a + b; v[k | h] = a - b; }
      const float lo[8] = {v[0], v[1], v[2], v[3], v[4], v[5], v[6], v[7]};
      const float hi[8] = {v[8], v[9], v[10], v[11], v[12], v[13], v[14], v[15]};
      store8(row, 0, lo, bs < 8 ? bs : 8);
      if (bs > 8) store8(row, 8, hi, bs - 8);
    }
    return;
  }
  const int row_words = bs + (bs >> 5);
  fht_tile_core(smem, logbs, rows, load32);
  const int plog = logbs - 3;                  // log2(8-value pieces per array)
  const int total = rows << plog;
  for (int o = threadIdx.x; o < total; o += blockDim.x) {
    const int row = o >> plog, i0 = (o & ((1 << plog) - 1)) << 3;
    const float* p = smem + row * row_words + fht_pad(i0);
    float v[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] = p[k];
    store8(row, i0, v, 8);
  }
}

// ---------------------------------------------------------------------------------------------------
// Low-latency transform of ONE array of 32 .. 8192 values by a 256-thread CTA, for the single-launch decode
// kernel where the transform sits on the critical path of a few-microsecond kernel: one round of global
// loads, one shared-memory exchange, one __syncthreads.
//   thread t holds E = max(1, bs / 256) consecutive values (index t * E + j): stages 0 .. log2(E) - 1 run in
//   registers, the next five across the lanes of a warp with shuffles, the last log2(W) (W = warps holding the
//   array, at most 8) after an exchange through shared memory, where a thread gathers the W values that differ
//   in the warp bits, finishes the butterflies and hands every finished value to `store(i, value)`; for a fixed
//   call of `store` the lanes of a warp hold consecutive i.
// Same butterflies in the same (ascending) order as fht_tile, so the results are bit-identical to it.
// `smem` needs bs + bs / 32 floats.  All 256 threads must call; `load(i0, v)` fills v[0..E) with values
// i0 .. i0 + E - 1.
// ---------------------------------------------------------------------------------------------------
template <int E, class Load, class Pre, class Store>
__device__ __forceinline__ void fht_fast_e(float* smem, int logbs, Load& load, Pre& pre, Store& store) {
  constexpr int LOGE = E == 1 ? 0 : E == 2 ? 1 : E == 4 ? 2 : E == 8 ? 3 : E == 16 ? 4 : 5;
  constexpr int QMAX = E >= 8 ? E / 8 : 1;         // rounds of the final loop (values per warp / 256)
  const int bs = 1 << logbs;
  const int t = threadIdx.x, lane = t & 31;
  const int nthreads = bs >> LOGE;                 // threads that hold values (32 .. 256)
  const int W = nthreads >> 5;                     // warps that hold values (1 .. 8)
  const bool active = t < nthreads;
  const int span = 32 << LOGE;                     // values per warp = distance between the W partners
  // What `store` needs besides the transformed value (a sign, the old output, ...) is requested first by
  // `pre(i)`, for exactly the indices this thread will store, so that it arrives while the transform runs.
  float aux[QMAX][8];
  if (W == 1) {
    if (active) {
#pragma unroll
      for (int j = 0; j < E; ++j) aux[0][j] = pre(t * E + j);        // E <= 1 here (32 values, one warp)
    }
  } else {
#pragma unroll
    for (int q = 0; q < QMAX; ++q) {
      const int r = t + 256 * q;
#pragma unroll
      for (int w = 0; w < 8; ++w) aux[q][w] = (r < span && w < W) ? pre(w * span + r) : 0.f;
    }
  }
  float v[E];
  if (active) {
    load(t * E, v);
    fht_regs<LOGE>(v);
#pragma unroll
    for (int k = 0; k < 5; ++k) {
      const bool upper = (lane >> k) & 1;
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const float p = __shfl_xor_sync(0xffffffffu, v[j], 1 << k);
        v[j] = upper ? (p - v[j]) : (v[j] + p);    // lower index: a + b, upper index: a - b (a = lower element)
      }
    }
  }
  if (W == 1) {
    if (active) {
#pragma unroll
      for (int j = 0; j < E; ++j) store(t * E + j, v[j], aux[0][j]);
    }
    return;
  }
  if (active) {
#pragma unroll
    for (int j = 0; j < E; ++j) smem[fht_pad(t * E + j)] = v[j];
  }
  __syncthreads();
  const int logw = W == 2 ? 1 : W == 4 ? 2 : 3;
#pragma unroll
  for (int q = 0; q < QMAX; ++q) {
    const int r = t + 256 * q;
    if (r < span) {
      float u[8];
#pragma unroll
      for (int w = 0; w < 8; ++w) u[w] = w < W ? smem[fht_pad(w * span + r)] : 0.f;
      if (logw == 1) {
        const float a = u[0], b = u[1];
        u[0] = a + b; u[1] = a - b;
      } else if (logw == 2) {
        float h[4] = {u[0], u[1], u[2], u[3]};
        fht_regs<2>(h);
        u[0] = h[0]; u[1] = h[1]; u[2] = h[2]; u[3] = h[3];
      } else {
        fht_regs<3>(u);
      }
#pragma unroll
      for (int w = 0; w < 8; ++w)
        if (w < W) store(w * span + r, u[w], aux[q][w]);
    }
  }
}

// dispatch on the array length (2^logbs, 32 .. 8192)
template <int MAXLOG = 13, class Load1, class Load4, class Pre, class Store>
__device__ __forceinline__ void fht_fast(float* smem, int logbs, Load1 load1, Load4 load4, Pre pre, Store store) {
  // load1(i) -> value i;  load4(i0, float (&q)[4]) -> values i0 .. i0 + 3 (i0 a multiple of 4);
  // pre(i) -> float handed back to store(i, value, that float)
  auto ld1 = [&](int i0, float (&v)[1]) { v[0] = load1(i0); };
  auto ld2 = [&](int i0, float (&v)[2]) { v[0] = load1(i0); v[1] = load1(i0 + 1); };
  auto ld4 = [&](int i0, float (&v)[4]) { load4(i0, v); };
  auto ld8 = [&](int i0, float (&v)[8]) {
    float q[4];
#pragma unroll
    for (int k = 0; k < 2; ++k) { load4(i0 + 4 * k, q); v[4 * k] = q[0]; v[4 * k + 1] = q[1]; v[4 * k + 2] = q[2]; v[4 * k + 3] = q[3]; }
  };
  auto ld16 = [&](int i0, float (&v)[16]) {
    float q[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) { load4(i0 + 4 * k, q); v[4 * k] = q[0]; v[4 * k + 1] = q[1]; v[4 * k + 2] = q[2]; v[4 * k + 3] = q[3]; }
  };
  auto ld32 = [&](int i0, float (&v)[32]) {
    float q[4];
#pragma unroll
    for (int k = 0; k < 8; ++k) { load4(i0 + 4 * k, q); v[4 * k] = q[0]; v[4 * k + 1] = q[1]; v[4 * k + 2] = q[2]; v[4 * k + 3] = q[3]; }
  };
  // arrays longer than 2^MAXLOG never reach this instantiation (their cases are not compiled)
  if (logbs == 9) { fht_fast_e<2>(smem, logbs, ld2, pre, store); return; }
  if (logbs == 10) { fht_fast_e<4>(smem, logbs, ld4, pre, store); return; }
  if constexpr (MAXLOG >= 11) if (logbs == 11) { fht_fast_e<8>(smem, logbs, ld8, pre, store); return; }
  if constexpr (MAXLOG >= 12) if (logbs == 12) { fht_fast_e<16>(smem, logbs, ld16, pre, store); return; }
  if constexpr (MAXLOG >= 13) if (logbs == 13) { fht_fast_e<32>(smem, logbs, ld32, pre, store); return; }
  fht_fast_e<1>(smem, logbs, ld1, pre, store);                        // 32 .. 256 values
}
constexpr int FHT_FAST_MAX_LOG = 13;

}  // namespace glqb
