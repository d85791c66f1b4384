/*
 * glq_b200 — C ABI of the B200 (sm_100a) compressed-weight matmul library for GLQ checkpoints.
 *
 * Everything here is plain C: device pointers travel as void*, sizes as integers, the CUDA
 * stream as an opaque pointer (a cudaStream_t).  The run entry points (glqb_plan_run, glqb_moe_plan_run,
 * glqb_input_rht, glqb_output_rht, glqb_output_rht_shards, the dump functions) allocate nothing, copy
 * nothing from host memory and do not synchronise: callers hand in a workspace (size reported by the
 * plan), so these calls may be captured into a CUDA graph.  Plan creation allocates a small device table;
 * glqb_fused_linear is a convenience wrapper that creates, runs and destroys a plan and synchronises.
 * Every function returns 0 on success or a negative GLQB_E_* code and never throws; glqb_last_error()
 * gives the message for the calling thread.
 *
 * Citations of the form file:line name the interface of the reference project (cnygaard/glq)
 * that the entry point stands in for.
 */
#ifndef GLQ_B200_H
#define GLQ_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GLQB_OK 0
#define GLQB_E_INVALID (-1)     /* bad argument / unsupported shape */
#define GLQB_E_CUDA (-2)        /* a CUDA runtime call failed */
#define GLQB_E_WORKSPACE (-3)   /* workspace missing or too small */
#define GLQB_E_DEVICE (-4)      /* kernel reported an internal error through its status word */

#define GLQB_FMT_TRELLIS_3INST 0   /* trellis_packed{,2}: glq/quantized_linear.py:351-361 */
#define GLQB_FMT_E8_SHELL 1        /* Qidxs{,2,3,4}:      glq/quantized_linear.py:235-247 */

#define GLQB_DT_F16 0
#define GLQB_DT_BF16 1
#define GLQB_DT_F32 2

#define GLQB_MAX_STAGES 4
#define GLQB_MAX_BLOCKS 16

/* Activation codes of the MoE ops (glq_vllm/fused_moe_method.py:671-677). */
#define GLQB_ACT_SILU 0
#define GLQB_ACT_GELU_TANH 1
#define GLQB_ACT_RELU2 2

/*
 * One quantised linear layer  y = [SU * H_m( wscale * W~ * H_n(SV * pad(x)) )][:out_features]
 * with W~ decoded on the fly from `codes`.  Mirrors the argument lists of
 *   glq_fused_linear_cuda / glq_fused_linear_block_diag_cuda    (glq/csrc/glq_bindings.cpp:334-550,
 *                                                                schemas glq_vllm/custom_ops.py:105-126)
 *   glq_fused_linear_trellis_3inst{,_rvq2}_cuda                 (glq_vllm/custom_ops.py:373-407)
 */
typedef struct GlqbLinearDesc {
  int32_t format;                        /* GLQB_FMT_* */
  int32_t m_pad, n_pad;                  /* stored matrix: rows (outputs) x cols (inputs) */
  int32_t in_features, out_features;     /* <= n_pad / <= m_pad */
  int32_t n_stages;                      /* trellis 1..2, E8 1..4 */
  int32_t bits[GLQB_MAX_STAGES];         /* trellis: K bits/weight of the stage (1..4); E8: unused */
  const void* codes[GLQB_MAX_STAGES];    /* device: int16 bit-stream / int16 index matrix per stage */
  const uint32_t* table[GLQB_MAX_STAGES];/* E8: device nibble-packed table of the stage (see glqb_e8_pack_table) */
  int32_t table_entries[GLQB_MAX_STAGES];/* E8: rows of that table (65536, or 256 for the small second stage) */
  float stage_scale[GLQB_MAX_STAGES];    /* [0] unused; [s] = cumulative inverse residual scale of stage s+1 */
  float wscale;                          /* the layer's scalar Wscale */
  const float* row_scale;                /* optional device fp32 (m_pad,) multiplied per output row of W~; NULL = none */
  const void* su;                        /* device fp16 (m_pad,) +-1 */
  const void* sv;                        /* device fp16 (n_pad,) +-1 */
  int32_t n_blocks_n, n_blocks_m;        /* block-diagonal Hadamard decomposition (powers of two, descending) */
  int32_t blocks_n[GLQB_MAX_BLOCKS];
  int32_t blocks_m[GLQB_MAX_BLOCKS];
  int32_t batch;                         /* tokens B (rows of x) */
  int32_t x_dtype, y_dtype;              /* GLQB_DT_* */
  int64_t x_stride, y_stride;            /* elements between consecutive tokens */
  int64_t x_offset, y_offset;            /* element offsets added to the x / y base pointers given at run time */
  int32_t stop_at_yrht;                  /* 1: write fp32 rotated-domain outputs (wscale applied, no output transform)
                                            to y (the "_yrht" ops, glq_vllm/custom_ops.py:388-392) */
  int32_t x_is_rotated;                  /* 1: x already holds H_n(SV * pad(x)) for n_pad columns (the unfused
                                            dequant_matvec / dequant_matmul ops, glq_vllm/custom_ops.py:58-71) */
  /* Optional fusions of the steps a decoder layer runs around its linears.  The reference has no such ops: its
   * callers launch RMSNorm, silu(gate) * up and the residual add as separate kernels between the GLQ ops
   * (glq_vllm/linear_method.py:1466; the host framework's decoder layer).  Served by the single-launch decode
   * form only (trellis, at most 8 tokens, every layer of the plan segment reading the same input): plan
   * creation refuses them otherwise, and callers then run those steps themselves. */
  const void* in_norm_weight;            /* RMSNorm weight (in_features,) of dtype in_norm_dtype, or NULL: the input becomes
                                            round(w * round(x * rsqrt(mean(x^2) + eps))), rounded to the x dtype */
  int32_t in_norm_dtype;                 /* GLQB_DT_* */
  float in_norm_eps;
  int32_t in_gated_act;                  /* 0: none; 1 + GLQB_ACT_{SILU,GELU_TANH,RELU2}: a row of x holds [gate | up]
                                            (2 * in_features values, x_stride apart); the input is
                                            round(round(act(gate)) * up), rounded to the x dtype */
  int32_t y_accumulate;                  /* 1: y <- y + result (residual add), y read in y_dtype */
} GlqbLinearDesc;

typedef struct GlqbPlan GlqbPlan;

/* Build a plan for `count` independent linears executed by ONE launch sequence (fused q/k/v or
 * gate/up shards that share x, the experts of one MoE step, or a whole sweep of layers).  Copies the
 * descriptors; uploads a small device table (the only allocation, at creation). */
int glqb_plan_create(const GlqbLinearDesc* descs, int32_t count, GlqbPlan** out_plan);
size_t glqb_plan_workspace_bytes(const GlqbPlan* plan);
/* algorithmic bytes (index / bit-stream tensors read once) and flops (2*B*m*n) of one run */
int64_t glqb_plan_code_bytes(const GlqbPlan* plan);
int64_t glqb_plan_flops(const GlqbPlan* plan);
/* kernels launched by one glqb_plan_run */
int32_t glqb_plan_launches(const GlqbPlan* plan);
/* Enqueue on `stream`; returns without synchronising.  x_base / y_base are device pointers the
 * descriptors' offsets are applied to. */
int glqb_plan_run(GlqbPlan* plan, const void* x_base, void* y_base,
                  void* workspace, size_t workspace_bytes, void* stream);
/* With timing enabled every run brackets its decode kernels with a CUDA event pair on the launching
 * stream.  glqb_plan_kernel_ms waits for those events and returns the summed kernel time (ms) and the
 * number of runs recorded since timing was (re-)enabled. */
int glqb_plan_set_timing(GlqbPlan* plan, int32_t enable);
int glqb_plan_kernel_ms(GlqbPlan* plan, double* total_ms_out, int32_t* runs_out);
/* Reads the plan's device status word (synchronising copy).  0 = every kernel of every run so far
 * completed normally; non-zero = a bounded wait inside a kernel expired (GLQB_E_DEVICE is returned). */
int glqb_plan_status(GlqbPlan* plan, int32_t* status_out);
void glqb_plan_destroy(GlqbPlan* plan);

/*
 * Sum over tensor-parallel ranks inside the kernels (one process per GPU, all on one node).  The reference leaves
 * the sum of row-parallel partial outputs (o_proj, down_proj) to its host framework's NCCL all-reduce
 * (glq_vllm/linear_method.py:1031-1102 runs under vLLM's RowParallelLinear); for decode-sized outputs that call is
 * all latency.  A communicator owns one receive area per rank, mapped into every rank (CUDA IPC); a CTA stores its
 * piece into all ranks' areas, raises a flag per peer, waits (bounded) for the peers' flags and adds the pieces in
 * rank order 0..G-1, so every rank gets the same bits.  No loads from peer memory, no bulk-tensor copies.
 *
 * Set-up, once: every rank calls glqb_comm_create (allocates its area: the only allocation), exchanges the
 * GLQB_COMM_HANDLE_BYTES handle of glqb_comm_handle with the other ranks by any host channel, and passes all ranks'
 * handles (rank order, `handle_stride` bytes apart) to glqb_comm_connect.  glqb_comm_connect_local is the same for
 * communicators that live in one process.  All ranks must then issue the same sequence of launches that use the
 * communicator (the protocol counts them on the device, so CUDA-graph replays need no changing argument).
 *
 * max_floats: fp32 values one launch may exchange per rank.  A wait that exceeds the time limit (default 2 s) sets
 * the status word instead of hanging: glqb_comm_status returns GLQB_E_DEVICE and the launch's results are invalid.
 */
typedef struct GlqbComm GlqbComm;
#define GLQB_COMM_HANDLE_BYTES 64
int glqb_comm_create(int32_t rank, int32_t world, int64_t max_floats, GlqbComm** out);
int glqb_comm_handle(GlqbComm* comm, void* handle_out, int32_t handle_bytes);
int glqb_comm_connect(GlqbComm* comm, const void* handles, int32_t handle_stride);
int glqb_comm_connect_local(GlqbComm* comm, GlqbComm* const* comms_by_rank);
int glqb_comm_set_timeout_ms(GlqbComm* comm, int32_t ms);
int64_t glqb_comm_max_floats(const GlqbComm* comm);
/* In-place sum of `count` fp32 values (count <= max_floats) over the ranks, one launch, no host synchronisation. */
int glqb_comm_all_reduce(GlqbComm* comm, void* buf_f32, int64_t count, void* stream);
/* Synchronising read of the status word; `reset` != 0 clears it afterwards. */
int glqb_comm_status(GlqbComm* comm, int32_t* status_out, int32_t reset);
/* launches that used the communicator so far (synchronising read; equal on all ranks between steps) */
int glqb_comm_epoch(GlqbComm* comm, int32_t* epoch_out);
void glqb_comm_destroy(GlqbComm* comm);
/* The outputs of all layers of `plan` become sums over the communicator's ranks, computed inside the single-launch
 * decode kernel right after the output transform (fp32, each rank with its own SU): every rank ends with the full
 * result, the residual add (y_accumulate) included.  Plans that do not take the single-launch form are refused with
 * GLQB_E_INVALID; sum their fp32 outputs with glqb_comm_all_reduce or NCCL instead.  comm = NULL detaches. */
int glqb_plan_set_comm(GlqbPlan* plan, GlqbComm* comm);

/*
 * MoE grouped expert matmul over trellis 3INST experts:
 *     out[t] = sum_j topk_weights[t,j] * W2_e( act( W13_e x_t ) ),  e = topk_ids[t,j]
 * Replaces glq_fused_moe_trellis_3inst_cuda (glq/csrc/glq_cuda.cu:5042; schema
 * glq_vllm/custom_ops.py:22-36) with the expert-stacked storage of glq_vllm/moe_shapes.py:56-72:
 * w13 = [gate; up] rows per expert, one SV per projection shared by all experts, SU / Wscale /
 * inv_resid_scale2 per expert.  Works for any token count (no 256-token cap, no host synchronisation).
 * The same plan type serves E8-shell experts (fields at the end of the struct).
 */
typedef struct GlqbMoeDesc {
  int32_t num_experts, top_k, hidden, inter, w13_out;
  int32_t max_tokens;                    /* capacity the workspace is sized for */
  int32_t activation;                    /* GLQB_ACT_* gated (0..2) or 3..5 = silu / gelu / relu^2 without gate */
  int32_t w13_bits, w13_bits2, w2_bits, w2_bits2;   /* K of stage 1 / stage 2 (bits2 ignored when packed2 is NULL) */
  const void* w13_packed;                /* (E, (w13_out/16)(hidden/16), 16K) int16 */
  const void* w13_packed2;               /* NULL when there is no second stage */
  const void* w13_su;                    /* (E, w13_out) fp16 */
  const void* w13_sv;                    /* (hidden,) fp16 */
  const float* w13_wscale;               /* (E,) fp32 device */
  const float* w13_inv_resid_scale2;     /* (E,) fp32 device, NULL without a second stage */
  const void* w2_packed;                 /* (E, (hidden/16)(inter/16), 16K) int16 */
  const void* w2_packed2;
  const void* w2_su;                     /* (E, hidden) fp16 */
  const void* w2_sv;                     /* (inter,) fp16 */
  const float* w2_wscale;
  const float* w2_inv_resid_scale2;
  int32_t n_blocks_n_w13, n_blocks_m_w13, n_blocks_n_w2, n_blocks_m_w2;
  int32_t blocks_n_w13[GLQB_MAX_BLOCKS], blocks_m_w13[GLQB_MAX_BLOCKS];
  int32_t blocks_n_w2[GLQB_MAX_BLOCKS], blocks_m_w2[GLQB_MAX_BLOCKS];
  int32_t ids_are_int64;                 /* topk_ids dtype: 1 = int64, 0 = int32 */
  int32_t x_dtype, y_dtype;              /* GLQB_DT_* */
  /* E8 shell experts: glq_fused_moe_grouped_gemm_cuda / glq_fused_moe_block_diag_cuda
   * (glq/csrc/glq_cuda.cu:4599, 5241; schemas glq_vllm/custom_ops.py:203-246; storage
   * glq_vllm/fused_moe_method.py:157-213).  With format == GLQB_FMT_E8_SHELL the trellis fields above
   * (w13_packed.., *_bits) are ignored; SU / SV / Wscale / blocks are shared with them. */
  int32_t format;                        /* GLQB_FMT_TRELLIS_3INST (0) or GLQB_FMT_E8_SHELL */
  int32_t e8_stages;                     /* 1..3 */
  const void* w13_qidxs[3];              /* per stage (E, w13_out, hidden/8) int16 */
  const void* w2_qidxs[3];               /* per stage (E, hidden, inter/8) int16 */
  const uint32_t* e8_table[3];           /* nibble-packed table of the stage (glqb_e8_pack_table) */
  int32_t e8_table_entries[3];
  const float* w13_inv_rs[2];            /* (E,) fp32 device: cumulative inverse residual scale of stages 2, 3 */
  const float* w2_inv_rs[2];
} GlqbMoeDesc;

typedef struct GlqbMoePlan GlqbMoePlan;
int glqb_moe_plan_create(const GlqbMoeDesc* desc, GlqbMoePlan** out_plan);
size_t glqb_moe_plan_workspace_bytes(const GlqbMoePlan* plan);
int64_t glqb_moe_plan_code_bytes(const GlqbMoePlan* plan);
/* x (tokens, hidden), topk_ids (tokens, top_k), topk_weights (tokens, top_k) fp32, y (tokens, hidden);
 * six or seven launches on `stream`, returns without synchronising.  Steps with at least 64 routed tokens
 * per expert on average (GLQB_MOE_GEMM_MIN_AVG) run the two matmuls on the tensor-core GEMM kernel. */
int glqb_moe_plan_run(GlqbMoePlan* plan, const void* x, const void* topk_ids, const float* topk_weights, void* y,
                      int32_t tokens, void* workspace, size_t workspace_bytes, void* stream);
/* Synchronises `stream` and reports whether a bounded wait inside the GEMM kernels of the last run gave up
 * (GLQB_E_DEVICE, results invalid); GLQB_OK otherwise.  No counterpart in the reference. */
int glqb_moe_plan_status(const GlqbMoePlan* plan, const void* workspace, void* stream);
/* With timing enabled every run brackets its two expert matmuls (w13, w2) with CUDA event pairs on the
 * launching stream; glqb_moe_plan_kernel_ms waits for them and returns the summed matmul time (ms) and the
 * number of runs recorded since timing was (re-)enabled.  No counterpart in the reference. */
int glqb_moe_plan_set_timing(GlqbMoePlan* plan, int32_t enable);
int glqb_moe_plan_kernel_ms(GlqbMoePlan* plan, double* total_ms_out, int32_t* runs_out);
void glqb_moe_plan_destroy(GlqbMoePlan* plan);

/* Stateless single-layer form of the reference's fused ops, for occasional calls: it builds a one-layer
 * plan, runs it, waits for `stream` and destroys the plan (so it allocates, synchronises and cannot be
 * captured).  `workspace` must hold glqb_linear_workspace_bytes(desc) bytes, a device-independent upper
 * bound of what the plan needs. */
size_t glqb_linear_workspace_bytes(const GlqbLinearDesc* desc);
int glqb_fused_linear(const GlqbLinearDesc* desc, const void* x, void* y,
                      void* workspace, size_t workspace_bytes, void* stream);

/* Kernel-internal decode written out, for the bit-exact gate.
 * Trellis: replaces glq_decompress_trellis_3inst_cuda (glq/csrc/glq_bindings.cpp:349-352) — one
 * stage gives fp16 (m, n); with a second stage the fp32 sum dec1 + dec2*inv_resid_scale2
 * (glq/trellis.py:923-933).  out_dtype GLQB_DT_F16 (single stage only) or GLQB_DT_F32. */
int glqb_decompress_trellis_3inst(const void* packed, int32_t bits, const void* packed2, int32_t bits2,
                                  float inv_resid_scale2, int32_t m, int32_t n,
                                  void* out, int32_t out_dtype, void* stream);
/* E8: W~ = cb[q1] + cb2[q2]*s1 + cb[q3]*s2 + cb[q4]*s3 evaluated left to right with separate fp32
 * multiply and add (glq/quantized_linear.py:1177-1194); out fp32 (m, n). */
int glqb_dequant_e8(const void* const* qidxs, const uint32_t* const* tables, const int32_t* table_entries,
                    const float* stage_scale, int32_t n_stages, int32_t m, int32_t n,
                    float* out, void* stream);
/* fp16 (entries, 8) codebook (the tensor the reference ops take, glq/codebook.py:189) -> nibble
 * packed uint32 (entries,) with nibble i = 2*coord_i + 6 (glq/codebook.py:102-115). */
int glqb_e8_pack_table(const void* codebook_f16, int32_t entries, uint32_t* out_packed, void* stream);

/* Unfused transforms: glq_input_rht_cuda / glq_output_rht_cuda (glq_vllm/custom_ops.py:90-99). */
int glqb_input_rht(const void* x, int32_t x_dtype, int64_t x_stride, const void* sv, void* out_f32,
                   int32_t in_features, int32_t n_pad, const int32_t* blocks, int32_t n_blocks,
                   int32_t batch, void* stream);
int glqb_output_rht(const float* y_rht, const void* su, void* out, int32_t out_dtype, int64_t out_stride,
                    int32_t out_features, int32_t m_pad, const int32_t* blocks, int32_t n_blocks,
                    int32_t batch, void* stream);

/* Output transform over the sub-blocks of several fused shards in one launch: glq_output_rht_shards_cuda
 * (glq/csrc/glq_cuda.cu:2882, schema glq_vllm/custom_ops.py:424-426).  y_rht is fp32 (batch, total_m);
 * block i covers columns [offsets[i], offsets[i] + blocks[i]) of y_rht, su and out.  At most
 * GLQB_MAX_BLOCKS blocks per call. */
int glqb_output_rht_shards(const float* y_rht, const void* su, void* out, int32_t out_dtype, int64_t out_stride,
                           int32_t out_features, int32_t total_m, const int32_t* offsets, const int32_t* blocks,
                           int32_t n_blocks, int32_t batch, void* stream);

/* glq_trellis_kernel_supported(m, k) (glq/csrc/glq_bindings.cpp:345). */
int glqb_trellis_kernel_supported(int32_t m, int32_t n);

/*
 * Batch-1 trellis 3INST linear (same mathematics as a one-layer plan) that needs neither a plan nor a
 * workspace: its scratch memory is a fixed array inside the library.  No counterpart in the reference.
 * It exists for callers that cannot allocate device memory where they run a layer (a host that sized
 * all device memory at start-up, a callback inside another allocator, a program without any
 * allocator of its own).  It calls no cudaMalloc/cudaFree and no allocating library routine.
 *   - limits: one token, one stage, K = 1..4, m % 32 == 0, n % 32 == 0, m and n <= 32768; larger or
 *     batched layers are refused with GLQB_E_INVALID (use the plan entry points);
 *   - glqb_noalloc_scratch_bytes() bytes (4 MiB) of device memory are held by every GPU that loads the
 *     library, until the process ends;
 *   - the first call on a device looks up the array's device address and raises two kernels'
 *     shared-memory limits: make that first call outside of any stream capture;
 *   - all calls on one GPU share the array (it keeps the previous call's contents; every word a
 *     call reads it has written earlier in the same call, so nothing needs clearing): calls that may
 *     overlap on the GPU — different streams, or different host threads — race and must be ordered
 *     by the caller.
 */
int glqb_trellis_linear_noalloc(const void* x, int32_t x_dtype, void* y, int32_t y_dtype, const void* packed,
                                int32_t bits, const void* su, const void* sv, float wscale, int32_t m, int32_t n,
                                const int32_t* blocks_n, int32_t n_blocks_n, const int32_t* blocks_m,
                                int32_t n_blocks_m, void* stream);
size_t glqb_noalloc_scratch_bytes(void);

const char* glqb_last_error(void);
const char* glqb_version(void);

#ifdef __cplusplus
}
#endif
#endif /* GLQ_B200_H */
