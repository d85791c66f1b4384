// Host-side launch interface between the plan builder (glqb_api.cu) and the translation units that
// instantiate the large kernel families (glqb_gemm_inst.cu: tensor-core GEMM and E8 tile decode;
// glqb_fused.cu: single-launch decode).  Splitting them keeps every unit's compile time in check.
#pragma once
#include "glqb_internal.h"
#include "glqb_comm.cuh"

namespace glqb {

struct GemmItem;

// One launch of a streaming decode kernel: a set of layers that share format / bit widths /
// token-column blocks, contiguous in the device table.
struct Segment {
  int format, k1, k2, ns, nb;
  int tn;                    // 0: streaming decode kernel; 128 / 256: tensor-core GEMM with that token tile
  int two_phase = 0;         // E8 GEMM with many tokens: weight tiles decoded once beforehand
  // single-launch form (input transform + decode + output transform in one kernel): all layers read one input
  bool fused = false;
  int total_units = 0, scratch_elems = 0;
  size_t fused_smem = 0;
  int first, count;          // range in the device table
  long long total_groups;
  int per_warp;
  int grid;
  int item_first, item_count;   // GEMM work items (range in the plan's item array)
  // E8 only: most of the codebook resident in shared memory (one CTA per SM)
  bool lut_table = false;    // trellis: table form of the streaming kernel (large batch-1 launches)
  bool smem_table = false;
  const uint32_t* big_table = nullptr;
  const uint32_t* small_table = nullptr;
  int small_entries = 0;
  int res_entries = 0;       // single-launch E8 form: table entries kept in shared memory (0: all gathers go to L1 / L2)
};


constexpr int GEMM_STAGES = 4;

// ---- glqb_gemm_inst.cu
bool gemm_available(const Segment& s);                       // is there a kernel for the segment's format / rates?
cudaError_t gemm_prepare(const Segment& s);                  // raises the kernel's dynamic shared-memory limit
cudaError_t tiles_smem_prepare(int ns);                      // same for the resident-table tile decode
// the segment's launches: (two-phase E8: tile decode, then) the GEMM over `items`
void gemm_launch(const Segment& s, const DevLinear* layers, const GemmItem* items, uint8_t* ws, int* status,
                 int sm_count, cudaStream_t stream);

// ---- glqb_fused.cu
bool fused_available(const Segment& s);                      // is there a single-launch kernel for the segment's format / rates?
cudaError_t fused_prepare(const Segment& s, size_t smem_limit, size_t smem, int* resident_ctas_out);
// `layers`: HOST copy of the segment's table entries (they are passed to the kernel by value)
// `comm`: null, or the communicator whose ranks' outputs are summed inside the kernel (layers with DevLinear::reduce)
void fused_launch(const Segment& s, const DevLinear* layers, const uint8_t* x_base, uint8_t* y_base, uint8_t* ws,
                  int* tickets, const CommDev* comm, cudaStream_t stream);

// ---- glqb_comm.cu
const CommDev* comm_dev(const GlqbComm* c);                  // null until the communicator is connected

}  // namespace glqb
