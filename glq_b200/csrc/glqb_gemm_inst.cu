// Instantiations and launches of the tensor-core GEMM kernels and the E8 tile decode (see glqb_gemm.cuh).
#include "glqb_kernels.cuh"
#include "glqb_gemm.cuh"
#include "glqb_launch.h"

namespace glqb {

typedef void (*TilesSmemKernel)(const DevLinear*, int, int, uint8_t*, const uint32_t*, const uint32_t*, int);
static TilesSmemKernel pick_tiles_smem_kernel(int ns) {
  switch (ns) {
    case 1: return e8_tiles_smem_kernel<1>;
    case 2: return e8_tiles_smem_kernel<2>;
    case 3: return e8_tiles_smem_kernel<3>;
    case 4: return e8_tiles_smem_kernel<4>;
  }
  return nullptr;
}

typedef void (*GemmKernel)(const DevLinear*, const GemmItem*, int, uint8_t*, int*, const int*);

template <int FORMAT, int K1, int K2>
static GemmKernel gemm_kernel_tn(int tn) {
  if (tn == 128) return glq_gemm_kernel<FORMAT, K1, K2, 128, GEMM_STAGES>;
  if (tn == 256) return glq_gemm_kernel<FORMAT, K1, K2, 256, GEMM_STAGES>;
  return nullptr;
}

typedef void (*TilesKernel)(const DevLinear*, int, int, uint8_t*);
static TilesKernel pick_tiles_kernel(int ns) {
  switch (ns) {
    case 1: return e8_tiles_kernel<1>;
    case 2: return e8_tiles_kernel<2>;
    case 3: return e8_tiles_kernel<3>;
    case 4: return e8_tiles_kernel<4>;
  }
  return nullptr;
}

static GemmKernel pick_gemm_kernel(const Segment& s) {
  if (s.two_phase) return gemm_kernel_tn<2, 0, 0>(s.tn);
  if (s.format == GLQB_FMT_TRELLIS_3INST) {
#define G_CASE(A, B) if (s.k1 == A && s.k2 == B) return gemm_kernel_tn<0, A, B>(s.tn);
#ifdef GLQB_FAST_BUILD   /* developer builds for kernel experiments: the 4-bit single-stage rate only */
    G_CASE(4, 0)
#else
    G_CASE(1, 0) G_CASE(2, 0) G_CASE(3, 0) G_CASE(4, 0)
    G_CASE(4, 1) G_CASE(4, 2) G_CASE(4, 3) G_CASE(4, 4)
#endif
  #undef G_CASE
    return nullptr;
  }
  switch (s.ns) {
    case 1: return gemm_kernel_tn<1, 1, 0>(s.tn);
    case 2: return gemm_kernel_tn<1, 2, 0>(s.tn);
    case 3: return gemm_kernel_tn<1, 3, 0>(s.tn);
    case 4: return gemm_kernel_tn<1, 4, 0>(s.tn);
  }
  return nullptr;
}

static size_t gemm_smem_bytes(int tn) {
  return (size_t)GEMM_STAGES * (GM_A_BYTES + (size_t)tn * 128) + (3 * GEMM_STAGES + 5) * 8 + 16 + 1024;
}


bool gemm_available(const Segment& s) { return pick_gemm_kernel(s) != nullptr; }

cudaError_t gemm_prepare(const Segment& s) {
  return cudaFuncSetAttribute(pick_gemm_kernel(s), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm_smem_bytes(s.tn));
}

cudaError_t tiles_smem_prepare(int ns) {
  return cudaFuncSetAttribute(pick_tiles_smem_kernel(ns), cudaFuncAttributeMaxDynamicSharedMemorySize, E8S_SMEM_BYTES);
}

void gemm_launch(const Segment& s, const DevLinear* layers, const GemmItem* items, uint8_t* ws, int* status,
                 int sm_count, cudaStream_t stream) {
  if (s.two_phase && s.smem_table)
    pick_tiles_smem_kernel(s.ns)<<<sm_count, E8TS_THREADS, E8S_SMEM_BYTES, stream>>>(
        layers, s.first, s.count, ws, s.big_table, s.small_table, s.small_entries);
  else if (s.two_phase)
    pick_tiles_kernel(s.ns)<<<sm_count * 8, 256, 0, stream>>>(layers, s.first, s.count, ws);
  pick_gemm_kernel(s)<<<s.grid, GM_THREADS, gemm_smem_bytes(s.tn), stream>>>(layers, items, s.item_count, ws, status, nullptr);
}

}  // namespace glqb
