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
