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

}  // namespace glqb
