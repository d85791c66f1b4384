// Instantiations and launches of the single-launch decode kernels (trellis_fused_kernel, e8_fused_kernel,
// glqb_kernels.cuh).
#include "glqb_kernels.cuh"
#include <cstdlib>
#include <cstring>

#include "glqb_launch.h"

namespace glqb {

typedef void (*FusedKernel)(const FusedLayers, int, int, int, const uint8_t*, uint8_t*, uint8_t*, int*, const CommDev);
static FusedKernel trellis_fused_pick(int k1, int k2) {
#define F_CASE(A, B) if (k1 == A && k2 == B) return trellis_fused_kernel<A, B>;
#ifdef GLQB_FAST_BUILD   /* developer builds for kernel experiments: the 4-bit single-stage rate only */
  F_CASE(4, 0)
#else
  F_CASE(1, 0) F_CASE(2, 0) F_CASE(3, 0) F_CASE(4, 0)
  F_CASE(4, 1) F_CASE(4, 2) F_CASE(4, 3) F_CASE(4, 4)
#endif
#undef F_CASE
  return nullptr;
}

typedef void (*E8FusedKernel)(const FusedLayers, int, int, int, const uint8_t*, uint8_t*, uint8_t*, int*, const CommDev,
                              const uint32_t*, int, const uint32_t*, int);
template <bool RES>
static E8FusedKernel e8_fused_pick_r(int ns) {
  switch (ns) {
    case 1: return e8_fused_kernel<1, RES>;
    case 2: return e8_fused_kernel<2, RES>;
#ifndef GLQB_FAST_BUILD
    case 3: return e8_fused_kernel<3, RES>;
    case 4: return e8_fused_kernel<4, RES>;
#endif
  }
  return nullptr;
}
static E8FusedKernel e8_fused_pick(int ns, bool res) { return res ? e8_fused_pick_r<true>(ns) : e8_fused_pick_r<false>(ns); }
static const void* fused_pick(const Segment& s) {
  if (s.format == GLQB_FMT_E8_SHELL) return reinterpret_cast<const void*>(e8_fused_pick(s.ns, s.res_entries > 0));
  return reinterpret_cast<const void*>(trellis_fused_pick(s.k1, s.k2));
}

bool fused_available(const Segment& s) { return fused_pick(s) != nullptr; }

cudaError_t fused_prepare(const Segment& s, size_t smem_limit, size_t smem, int* resident_ctas_out) {
  const void* fk = fused_pick(s);
  cudaError_t e = cudaFuncSetAttribute(fk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_limit);
  if (e != cudaSuccess) return e;
  return cudaOccupancyMaxActiveBlocksPerMultiprocessor(resident_ctas_out, fk, MV_THREADS, smem);
}

void fused_launch(const Segment& s, const DevLinear* layers, const uint8_t* x_base, uint8_t* y_base, uint8_t* ws,
                  int* tickets, const CommDev* comm, cudaStream_t stream) {
  // Launched with programmatic stream serialization: when the previous kernel of the stream is another
  // single-launch decode kernel, this one's prologue (scheduling, table reads, the first weight loads) overlaps
  // its tail; the kernel itself waits (griddepcontrol.wait) before it reads activations or writes anything.
  static const bool pdl = [] { const char* e = getenv("GLQB_PDL"); return !e || atoi(e) != 0; }();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)s.grid);
  cfg.blockDim = dim3(MV_THREADS);
  cfg.dynamicSmemBytes = s.fused_smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  FusedLayers T;
  memcpy(T.L, layers, sizeof(DevLinear) * (size_t)s.count);          // `layers`: the plan's HOST copy of the segment's entries
  CommDev C;
  memset(&C, 0, sizeof(C));                                           // world 0: no sum over ranks
  if (comm) C = *comm;
  if (s.format == GLQB_FMT_E8_SHELL) {
    cudaLaunchKernelEx(&cfg, e8_fused_pick(s.ns, s.res_entries > 0), T, s.count, s.total_units, s.scratch_elems, x_base, y_base,
                       ws, tickets, C, s.big_table, s.res_entries, s.small_table, s.small_entries);
    return;
  }
  cudaLaunchKernelEx(&cfg, trellis_fused_pick(s.k1, s.k2), T, s.count, s.total_units, s.scratch_elems, x_base, y_base, ws,
                     tickets, C);
}

}  // namespace glqb
