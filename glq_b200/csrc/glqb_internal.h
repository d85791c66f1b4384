// Internal structures shared by the host-side plan builder and the kernels.
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "../../include/glq_b200.h"

namespace glqb {

// Device-side description of one linear layer inside a plan.  Pointers into the caller's
// workspace are stored as byte offsets so that the workspace may move between runs.
struct DevLinear {
  const uint8_t* codes[GLQB_MAX_STAGES];
  const uint32_t* table[GLQB_MAX_STAGES];
  const __half* su;
  const __half* sv;
  const float* row_scale;
  float stage_scale[GLQB_MAX_STAGES];
  float wscale;
  int table_entries[GLQB_MAX_STAGES];
  int format, m, n, in_f, out_f, n_stages;
  int bits[GLQB_MAX_STAGES];
  int batch, x_dtype, y_dtype, stop_at_yrht, x_is_rotated;
  long long x_stride, y_stride, x_off, y_off;
  long long xr_off;      // workspace bytes: rotated activations, fp16 [batch][n]
  long long part_off;    // workspace bytes: partial sums, fp32 [slots][batch][m]
  long long atile_off;   // workspace bytes: pre-decoded fp16 weight tiles (two-phase E8 prefill), else unused
  long long group_base;  // first work-group index of this layer inside its launch segment
  int groups_per_strip;  // work groups along one strip of rows
  int strips;            // strips of rows (trellis: 32 rows, E8: 16 rows)
  int slots;             // upper bound on partial sums per strip
  int per_warp;          // work groups handed to each warp of the segment's launch
  int fixed_slots;       // > 0: every strip has exactly this many partial sums (GEMM path: K splits)
  int gemm_tn;           // token tile of the GEMM path (0: streaming decode path)
  int ticket_base;       // single-launch form: first completion ticket of this layer (one per output Hadamard block)
  const void* in_norm_w; // optional fusions (single-launch form): RMSNorm weight, its dtype and epsilon,
  int in_norm_dtype;     // gated activation of a [gate | up] input (0 none, 1 + GLQB_ACT_*), residual accumulate
  float in_norm_eps;
  int in_gated_act;
  int y_accumulate;
  int xr_global;         // single-launch form, wide inputs: the transformed activations come from the workspace
                         // (written by rht_in_kernel just before) instead of being recomputed by every CTA
  long long rstd_off;    // workspace bytes: 1 / rms of every token (fused RMSNorm applied to the output), written by the
                         // single-launch kernel for the output transforms that run as a kernel of their own
  int out_split_log;     // single-launch form: output blocks of at least 2^this rows are transformed by rht_out_kernel
  int reduce;            // single-launch form, tensor-parallel ranks: the output is summed over the ranks in the kernel
  int comm_off;          // ... first float of this layer's pieces in the receive areas, and its first piece number
  int comm_unit_base;
  int nbn, nbm;
  int bn_off[GLQB_MAX_BLOCKS], bn_log[GLQB_MAX_BLOCKS];
  int bm_off[GLQB_MAX_BLOCKS], bm_log[GLQB_MAX_BLOCKS];
};

// One (layer, Hadamard block) pair handled by one CTA of the transform kernels.
struct RhtItem {
  int layer;
  int block;
  int tok0;    // first token of the tile this CTA transforms
  int ntok;    // tokens in the tile (the CTA's shared memory holds ntok * block floats)
  int sub;     // -1: the whole block.  k >= 0 (decode-sized plans, blocks of 4096 values or more): the CTA produces
               // the k-th run of 1024 outputs only, as H_1024( sum_k' H_S[k][k'] * input run k' ) — H_(S*1024) =
               // H_S (x) H_1024 with the short factor applied first, so S CTAs share a long block without talking
};

#ifndef GLQB_RHT_TILE
#define GLQB_RHT_TILE 8192
#endif
// tokens per CTA of the transform kernels: about GLQB_RHT_TILE floats of shared memory per CTA
static inline int rht_tile_tokens(int block_size, int batch) {
  int t = GLQB_RHT_TILE / block_size;
  if (t < 1) t = 1;
  if (t > 64) t = 64;
  return t < batch ? t : batch;
}

// Stores the message glqb_last_error() returns for the calling thread (defined in glqb_api.cu).
void set_error_message(const char* msg);

// Status word of a plan: 0 = every kernel finished normally.  A role of the GEMM kernel whose bounded wait
// ran out writes its code here (never a trap): 2 producers, 3 MMA issuer, 4 activation loader, 5 epilogue.
// 6: a wait for a tensor-parallel peer ran out (communicator status word, glqb_comm.cuh).
enum : int { ST_OK = 0, ST_GAVE_UP_PRODUCER = 2, ST_GAVE_UP_MMA = 3, ST_GAVE_UP_LOADER = 4, ST_GAVE_UP_EPILOGUE = 5, ST_GAVE_UP_PEER = 6 };

}  // namespace glqb
