// C ABI of libglq_b200: plan builder, launch sequencing, stateless wrappers.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

#include "glqb_kernels.cuh"
#include "glqb_gemm.cuh"
#include "glqb_launch.h"

namespace glqb {

static thread_local std::string g_err;

void set_error_message(const char* msg) { g_err = msg ? msg : ""; }

static int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

#define CUDA_TRY(expr)                                                                   \
  do {                                                                                   \
    cudaError_t _e = (expr);                                                             \
    if (_e != cudaSuccess) return fail(GLQB_E_CUDA, "%s: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static inline int ilog2(int v) { int l = 0; while ((1 << l) < v) ++l; return l; }

constexpr int DECODE_MAX_BATCH = 64;   // above this the GEMM path is used

}  // namespace glqb

using namespace glqb;

struct GlqbPlan {
  std::vector<GlqbLinearDesc> descs;   // in caller order
  std::vector<int> order;              // device-table position -> caller index
  std::vector<DevLinear> dev;          // host copy of the device table
  std::vector<Segment> segs;
  std::vector<RhtItem> items_in, items_out;
  std::vector<RhtItem> items_in_gemm;
  std::vector<GemmItem> gemm_items;
  DevLinear* d_layers = nullptr;
  RhtItem* d_items_in = nullptr;
  RhtItem* d_items_in_gemm = nullptr;
  RhtItem* d_items_out = nullptr;
  GemmItem* d_gemm_items = nullptr;
  int* d_status = nullptr;
  int* d_tickets = nullptr;      // completion tickets of the single-launch form, all zero between runs
  const GlqbComm* comm = nullptr;  // tensor-parallel ranks whose outputs the single-launch kernel sums (glqb_plan_set_comm)
  int n_tickets = 0;
  int max_batch_gemm = 1;
  size_t ws_bytes = 0;
  int max_batch = 1;
  int max_bs_in = 32, max_bs_out = 32;
  int max_elems_in = 32, max_elems_out = 32;    // floats of shared memory the transform CTAs need
  int sm_count = 0;
  int64_t code_bytes = 0, flops = 0;
  bool timing = false;
  std::vector<cudaEvent_t> ev;   // pairs (start, stop) around the decode kernels of each timed run
  size_t ev_used = 0;
};

namespace glqb {

// ------------------------------------------------------------------------------------------
// kernel variant tables
// ------------------------------------------------------------------------------------------
typedef void (*MvKernel)(const DevLinear*, int, long long, int, uint8_t*);

template <int K1, int K2>
static MvKernel trellis_kernel_nb(int nb) {
  switch (nb) {
    case 1: return trellis_mv_kernel<K1, K2, 1>;
    case 2: return trellis_mv_kernel<K1, K2, 2>;
    case 4: return trellis_mv_kernel<K1, K2, 4>;
    case 8: if constexpr (K2 == 0) return trellis_mv_kernel<K1, K2, 8>; else return nullptr;
  }
  return nullptr;
}

// table form of the single-stage batch-1 kernels (large launches only)
static MvKernel trellis_lut_kernel(int k1) {
  switch (k1) {
#ifndef GLQB_FAST_BUILD
    case 2: return trellis_mv_kernel<2, 0, 1, MV_LUT_STATES>;
    case 3: return trellis_mv_kernel<3, 0, 1, MV_LUT_STATES>;
#endif
    case 4: return trellis_mv_kernel<4, 0, 1, MV_LUT_STATES>;
  }
  return nullptr;
}
static long long trellis_lut_min_bytes() {
  // every CTA spends a microsecond or two filling its table, so small launches keep the arithmetic decode
  const char* e = getenv("GLQB_TRELLIS_LUT_MIN_BYTES");
  return e ? atoll(e) : (48ll << 20);
}

static MvKernel trellis_kernel(int k1, int k2, int nb) {
#define T_CASE(A, B) if (k1 == A && k2 == B) return trellis_kernel_nb<A, B>(nb);
#ifdef GLQB_FAST_BUILD   /* developer builds for kernel experiments: the 4-bit single-stage rate only */
  T_CASE(4, 0)
#else
  T_CASE(1, 0) T_CASE(2, 0) T_CASE(3, 0) T_CASE(4, 0)
  T_CASE(4, 1) T_CASE(4, 2) T_CASE(4, 3) T_CASE(4, 4)
#endif
#undef T_CASE
  return nullptr;
}

template <int NS>
static MvKernel e8_kernel_nb(int nb) {
  switch (nb) {
    case 1: return e8_mv_kernel<NS, 1>;
    case 2: return e8_mv_kernel<NS, 2>;
    case 4: return e8_mv_kernel<NS, 4>;
    case 8: if constexpr (NS <= 2) return e8_mv_kernel<NS, 8>; else return nullptr;
  }
  return nullptr;
}

static MvKernel e8_kernel(int ns, int nb) {
  switch (ns) {
    case 1: return e8_kernel_nb<1>(nb);
    case 2: return e8_kernel_nb<2>(nb);
    case 3: return e8_kernel_nb<3>(nb);
    case 4: return e8_kernel_nb<4>(nb);
  }
  return nullptr;
}

constexpr size_t FUSED_SMEM_LIMIT = 200 * 1024;
constexpr size_t FUSED_SMEM_MAX = 226 * 1024;       // one CTA per SM (the E8 form with a resident codebook); 1 KB left for static shared memory
static bool fused_enabled() {
  const char* e = getenv("GLQB_FUSED_DECODE");
  return !e || atoi(e) != 0;
}
// do two layers read the same transformed input?
static bool same_input(const GlqbLinearDesc& a, const GlqbLinearDesc& b) {
  return a.in_norm_weight == b.in_norm_weight && a.in_norm_dtype == b.in_norm_dtype && a.in_norm_eps == b.in_norm_eps &&
         a.in_gated_act == b.in_gated_act &&
         a.format == b.format && a.n_pad == b.n_pad && a.in_features == b.in_features && a.sv == b.sv &&
         a.batch == b.batch && a.x_offset == b.x_offset && a.x_stride == b.x_stride && a.x_dtype == b.x_dtype &&
         a.x_is_rotated == b.x_is_rotated && a.n_blocks_n == b.n_blocks_n &&
         memcmp(a.blocks_n, b.blocks_n, sizeof(int32_t) * a.n_blocks_n) == 0;
}

typedef void (*E8SmemKernel)(const DevLinear*, int, long long, int, uint8_t*, const uint32_t*, const uint32_t*, int);

template <int NS>
static E8SmemKernel e8_smem_kernel_nb(int nb) {
  switch (nb) {
    case 1: return e8_mv_smem_kernel<NS, 1>;
    case 2: return e8_mv_smem_kernel<NS, 2>;
    case 4: if constexpr (NS <= 2) return e8_mv_smem_kernel<NS, 4>; else return nullptr;
  }
  return nullptr;
}

static E8SmemKernel pick_e8_smem_kernel(const Segment& s) {
  switch (s.ns) {
    case 1: return e8_smem_kernel_nb<1>(s.nb);
    case 2: return e8_smem_kernel_nb<2>(s.nb);
    case 3: return e8_smem_kernel_nb<3>(s.nb);
    case 4: return e8_smem_kernel_nb<4>(s.nb);
  }
  return nullptr;
}

#ifndef GLQB_E8_SMEM_MAX_NB
#define GLQB_E8_SMEM_MAX_NB 2      // token-column blocks up to which the resident-table kernel is used
#endif
static long long e8_smem_min_bytes() {
  const char* e = getenv("GLQB_E8_SMEM_MIN_BYTES");
  // Filling the table costs every CTA about 224 KiB of L2 reads per launch (a few microseconds), so small
  // launches keep the global-memory gathers.
  return e ? atoll(e) : (48ll << 20);
}

// Do all layers of the segment read one 65,536-entry table (and at most one small table)?  Also sums the
// index bytes of the segment.
static bool e8_uniform_tables(const std::vector<DevLinear>& dev, const Segment& s, const uint32_t** big_out,
                              const uint32_t** small_out, int* small_n_out, long long* bytes_out) {
  long long bytes = 0;
  const uint32_t* big = nullptr;
  const uint32_t* small = nullptr;
  int small_n = 0;
  for (int i = 0; i < s.count; ++i) {
    const DevLinear& L = dev[s.first + i];
    bytes += (long long)L.n_stages * L.m * (L.n / 8) * 2;
    for (int st = 0; st < L.n_stages; ++st) {
      if (L.table_entries[st] == 65536) {
        if (big && big != L.table[st]) return false;
        big = L.table[st];
      } else if (L.table_entries[st] <= 256) {
        if (small && (small != L.table[st] || small_n != L.table_entries[st])) return false;
        small = L.table[st];
        small_n = L.table_entries[st];
      } else {
        return false;
      }
    }
  }
  *big_out = big; *small_out = small; *small_n_out = small_n; *bytes_out = bytes;
  return big != nullptr;
}

static MvKernel pick_kernel(const Segment& s) {
  return s.format == GLQB_FMT_TRELLIS_3INST ? trellis_kernel(s.k1, s.k2, s.nb) : e8_kernel(s.ns, s.nb);
}

// token count from which E8 prefill decodes the weight tiles once instead of once per token tile
static int e8_two_phase_min_tokens() {
  const char* e = getenv("GLQB_E8_TWO_PHASE_MIN_TOKENS");
  return e ? atoi(e) : 129;     // measured on B200: above one 128-token tile the tile decode plus a copy-fed GEMM wins
}

static int tn_for_batch(int batch) { return batch <= DECODE_MAX_BATCH ? 0 : (batch <= 128 ? 128 : 256); }

static int nb_for_batch(int batch) {
  if (batch <= 8) return 1;
  if (batch <= 16) return 2;
  if (batch <= 32) return 4;
  return 8;
}

static int validate(const GlqbLinearDesc& d, int idx) {
  if (d.format != GLQB_FMT_TRELLIS_3INST && d.format != GLQB_FMT_E8_SHELL)
    return fail(GLQB_E_INVALID, "layer %d: unknown format %d", idx, d.format);
  if (d.m_pad <= 0 || d.n_pad <= 0 || d.in_features <= 0 || d.out_features <= 0 ||
      d.in_features > d.n_pad || d.out_features > d.m_pad)
    return fail(GLQB_E_INVALID, "layer %d: bad dims m_pad=%d n_pad=%d in=%d out=%d", idx, d.m_pad, d.n_pad,
                d.in_features, d.out_features);
  if (d.batch < 1) return fail(GLQB_E_INVALID, "layer %d: batch %d", idx, d.batch);
  if (d.batch > 65535) return fail(GLQB_E_INVALID, "layer %d: batch %d exceeds 65535 tokens", idx, d.batch);
  if (!d.su || !d.sv || !d.codes[0]) return fail(GLQB_E_INVALID, "layer %d: null su/sv/codes", idx);
  // the kernels read the sign vectors and the trellis bit-streams with 16-byte accesses
  if ((reinterpret_cast<uintptr_t>(d.su) | reinterpret_cast<uintptr_t>(d.sv)) & 15)
    return fail(GLQB_E_INVALID, "layer %d: su / sv must be 16-byte aligned", idx);
  if (d.format == GLQB_FMT_TRELLIS_3INST) {
    if (d.m_pad % 32 || d.n_pad % 32)
      return fail(GLQB_E_INVALID, "layer %d: trellis needs m %% 32 == 0 and n %% 32 == 0 (got %d x %d)", idx,
                  d.m_pad, d.n_pad);
    if (d.n_stages < 1 || d.n_stages > 2) return fail(GLQB_E_INVALID, "layer %d: trellis stages %d", idx, d.n_stages);
    for (int s = 0; s < d.n_stages; ++s)
      if (d.bits[s] < 1 || d.bits[s] > 4 || !d.codes[s])
        return fail(GLQB_E_INVALID, "layer %d: trellis stage %d has K=%d (supported 1..4)", idx, s, d.bits[s]);
    for (int s = 0; s < d.n_stages; ++s)
      if (reinterpret_cast<uintptr_t>(d.codes[s]) & 15)
        return fail(GLQB_E_INVALID, "layer %d: trellis stage %d bit-stream must be 16-byte aligned", idx, s);
    if (!trellis_kernel(d.bits[0], d.n_stages > 1 ? d.bits[1] : 0, 1))
      return fail(GLQB_E_INVALID, "layer %d: no kernel for trellis rates K=%d+%d", idx, d.bits[0],
                  d.n_stages > 1 ? d.bits[1] : 0);
    if (d.in_features != d.n_pad) return fail(GLQB_E_INVALID, "layer %d: trellis layers are never padded", idx);
  } else {
    if (d.n_pad % 8) return fail(GLQB_E_INVALID, "layer %d: E8 needs n_pad %% 8 == 0", idx);
    if (d.n_stages < 1 || d.n_stages > 4) return fail(GLQB_E_INVALID, "layer %d: E8 stages %d", idx, d.n_stages);
    for (int s = 0; s < d.n_stages; ++s) {
      if (!d.codes[s] || !d.table[s]) return fail(GLQB_E_INVALID, "layer %d: E8 stage %d null codes/table", idx, s);
      if ((reinterpret_cast<uintptr_t>(d.codes[s]) & 1) || (reinterpret_cast<uintptr_t>(d.table[s]) & 15))
        return fail(GLQB_E_INVALID, "layer %d: E8 stage %d misaligned index matrix (2 bytes) or table (16 bytes)", idx, s);
      const int e = d.table_entries[s];
      if (e < 1 || e > 65536 || (e & (e - 1)))
        return fail(GLQB_E_INVALID, "layer %d: E8 table entries %d must be a power of two <= 65536", idx, e);
    }
  }
  int sn = 0, sm = 0;
  if (d.n_blocks_n < 1 || d.n_blocks_n > GLQB_MAX_BLOCKS || d.n_blocks_m < 1 || d.n_blocks_m > GLQB_MAX_BLOCKS)
    return fail(GLQB_E_INVALID, "layer %d: block counts %d/%d", idx, d.n_blocks_n, d.n_blocks_m);
  for (int i = 0; i < d.n_blocks_n; ++i) {
    const int b = d.blocks_n[i];
    if (b < 1 || (b & (b - 1)) || b > 32768) return fail(GLQB_E_INVALID, "layer %d: blocks_n[%d]=%d", idx, i, b);
    sn += b;
  }
  for (int i = 0; i < d.n_blocks_m; ++i) {
    const int b = d.blocks_m[i];
    if (b < 1 || (b & (b - 1)) || b > 32768) return fail(GLQB_E_INVALID, "layer %d: blocks_m[%d]=%d", idx, i, b);
    sm += b;
  }
  if (sn != d.n_pad || sm != d.m_pad)
    return fail(GLQB_E_INVALID, "layer %d: Hadamard blocks sum to %d/%d, expected n_pad=%d m_pad=%d", idx, sn, sm,
                d.n_pad, d.m_pad);
  if (d.x_dtype < 0 || d.x_dtype > 2 || d.y_dtype < 0 || d.y_dtype > 2)
    return fail(GLQB_E_INVALID, "layer %d: dtype", idx);
  if (d.stop_at_yrht && d.y_dtype != GLQB_DT_F32)
    return fail(GLQB_E_INVALID, "layer %d: rotated-domain output must be fp32", idx);
  if (d.in_gated_act < 0 || d.in_gated_act > 3 || (d.in_norm_weight && (d.in_norm_dtype < 0 || d.in_norm_dtype > 2)))
    return fail(GLQB_E_INVALID, "layer %d: input activation code %d / norm weight dtype %d", idx, d.in_gated_act, d.in_norm_dtype);
  if ((d.in_gated_act || d.in_norm_weight) && d.x_is_rotated)
    return fail(GLQB_E_INVALID, "layer %d: input fusions need an untransformed input", idx);
  if (d.y_accumulate && d.stop_at_yrht)
    return fail(GLQB_E_INVALID, "layer %d: the residual add applies to the final output only", idx);
  return GLQB_OK;
}

// packed bytes of a layer's codes (what a decode launch must read once)
static long long layer_code_bytes(const GlqbLinearDesc& d) {
  if (d.format == GLQB_FMT_TRELLIS_3INST) {
    long long b = 0;
    for (int s = 0; s < d.n_stages; ++s) b += (long long)d.m_pad * d.n_pad * d.bits[s] / 8;
    return b;
  }
  return (long long)d.n_stages * d.m_pad * (d.n_pad / 8) * 2;
}

// one thread per 32-value segment of the largest tile, between 64 and RHT_THREADS
// ... except for decode-sized plans (at most 8 tokens), whose transforms use all 256 threads per array
static int rht_threads(int max_elems, int max_batch = 1 << 30) {
  if (max_batch <= FUSED_MAX_TOKENS) return RHT_THREADS;
  return std::max(64, std::min(RHT_THREADS, (max_elems / 32 + 31) / 32 * 32));
}
static int rht_smem(int max_elems) { return (max_elems + max_elems / 32) * 4 + 64; }

static cudaError_t raise_rht_smem_limits() {
  const int lim = rht_smem(32768);
  cudaError_t e = cudaFuncSetAttribute(rht_in_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(rht_in_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(rht_in_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(rht_out_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(rht_out_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
  return e;
}

// one item per (layer, block, tile of tokens); tracks the largest tile (floats) for the launch's smem.
// Decode-sized layers (at most 8 tokens): a block of 4096 values or more is shared by S = bs / 1024 CTAs, each
// producing one run of 1024 outputs for all tokens (RhtItem::sub).  `min_log`: only blocks of at least
// 2^min_log values get items (the single-launch kernel transforms the shorter output blocks itself).
static void add_rht_items(std::vector<RhtItem>& items, int layer, int nblocks, const int* logs, int batch,
                          int& max_elems, bool latency, int min_log = 0) {
  for (int b = 0; b < nblocks; ++b) {
    if (logs[b] < min_log) continue;
    const int bs = 1 << logs[b];
    if (latency && batch <= FUSED_MAX_TOKENS && logs[b] >= RHT_SPLIT_MIN_LOG) {
      for (int k = 0; k < (bs >> RHT_SPLIT_LOG); ++k) items.push_back(RhtItem{layer, b, 0, batch, k});
      max_elems = std::max(max_elems, 1 << RHT_SPLIT_LOG);
      continue;
    }
    const int tt = rht_tile_tokens(bs, batch);
    for (int t0 = 0; t0 < batch; t0 += tt) {
      const int nt = std::min(tt, batch - t0);
      items.push_back(RhtItem{layer, b, t0, nt, -1});
      max_elems = std::max(max_elems, nt * bs);
    }
  }
}

static int build_plan(GlqbPlan* P) {
  const int n = (int)P->descs.size();
  int dev_id = 0;
  CUDA_TRY(cudaGetDevice(&dev_id));
  CUDA_TRY(cudaDeviceGetAttribute(&P->sm_count, cudaDevAttrMultiProcessorCount, dev_id));

  // ---- segments: layers with the same kernel variant, in caller order inside a segment
  typedef std::tuple<int, int, int, int, int, int, int> Key;   // format, k1, k2, ns, nb, tn, two-phase
  std::map<Key, std::vector<int>> groups;
  std::vector<Key> key_order;
  for (int i = 0; i < n; ++i) {
    const GlqbLinearDesc& d = P->descs[i];
    Key k;
    const int tn = tn_for_batch(d.batch);
    const int nb = tn ? 0 : nb_for_batch(d.batch);
    if (d.format == GLQB_FMT_TRELLIS_3INST)
      k = Key(d.format, d.bits[0], d.n_stages > 1 ? d.bits[1] : 0, d.n_stages, nb, tn, 0);
    else
      k = Key(d.format, 0, 0, d.n_stages, nb, tn, (tn && d.batch >= e8_two_phase_min_tokens()) ? 1 : 0);
    if (!groups.count(k)) key_order.push_back(k);
    groups[k].push_back(i);
  }
  P->order.clear();
  P->segs.clear();
  for (const Key& k : key_order) {
    Segment s;
    s.format = std::get<0>(k); s.k1 = std::get<1>(k); s.k2 = std::get<2>(k);
    s.ns = std::get<3>(k); s.nb = std::get<4>(k); s.tn = std::get<5>(k); s.two_phase = std::get<6>(k);
    s.item_first = s.item_count = 0;
    s.first = (int)P->order.size();
    s.count = (int)groups[k].size();
    for (int i : groups[k]) P->order.push_back(i);
    if (s.tn ? !gemm_available(s) : !pick_kernel(s))
      return fail(GLQB_E_INVALID, "no kernel variant for format=%d K=%d+%d stages=%d token blocks=%d", s.format,
                  s.k1, s.k2, s.ns, s.nb);
    P->segs.push_back(s);
  }

  // ---- device table
  P->dev.assign(n, DevLinear());
  P->code_bytes = 0;
  P->flops = 0;
  P->max_batch = 1;
  for (int pos = 0; pos < n; ++pos) {
    const GlqbLinearDesc& d = P->descs[P->order[pos]];
    DevLinear& L = P->dev[pos];
    memset(&L, 0, sizeof L);
    for (int s = 0; s < GLQB_MAX_STAGES; ++s) {
      L.codes[s] = reinterpret_cast<const uint8_t*>(d.codes[s]);
      L.table[s] = d.table[s];
      L.table_entries[s] = d.table_entries[s];
      L.stage_scale[s] = d.stage_scale[s];
      L.bits[s] = d.bits[s];
    }
    L.su = reinterpret_cast<const __half*>(d.su);
    L.sv = reinterpret_cast<const __half*>(d.sv);
    L.row_scale = d.row_scale;
    L.wscale = d.wscale;
    L.format = d.format; L.m = d.m_pad; L.n = d.n_pad; L.in_f = d.in_features; L.out_f = d.out_features;
    L.n_stages = d.n_stages;
    L.batch = d.batch; L.x_dtype = d.x_dtype; L.y_dtype = d.y_dtype; L.stop_at_yrht = d.stop_at_yrht; L.x_is_rotated = d.x_is_rotated;
    L.x_stride = d.x_stride; L.y_stride = d.y_stride; L.x_off = d.x_offset; L.y_off = d.y_offset;
    L.in_norm_w = d.in_norm_weight; L.in_norm_dtype = d.in_norm_dtype; L.in_norm_eps = d.in_norm_eps;
    L.in_gated_act = d.in_gated_act; L.y_accumulate = d.y_accumulate;
    L.nbn = d.n_blocks_n; L.nbm = d.n_blocks_m;
    int off = 0;
    for (int i = 0; i < d.n_blocks_n; ++i) {
      L.bn_off[i] = off; L.bn_log[i] = ilog2(d.blocks_n[i]); off += d.blocks_n[i];
      P->max_bs_in = std::max(P->max_bs_in, d.blocks_n[i]);
    }
    off = 0;
    for (int i = 0; i < d.n_blocks_m; ++i) {
      L.bm_off[i] = off; L.bm_log[i] = ilog2(d.blocks_m[i]); off += d.blocks_m[i];
      P->max_bs_out = std::max(P->max_bs_out, d.blocks_m[i]);
    }
    if (d.format == GLQB_FMT_TRELLIS_3INST) {
      L.groups_per_strip = d.n_pad / 32;
      L.strips = d.m_pad / 32;
      for (int s = 0; s < d.n_stages; ++s) P->code_bytes += (int64_t)d.m_pad * d.n_pad * d.bits[s] / 8;
    } else {
      L.groups_per_strip = (d.n_pad + 255) / 256;
      L.strips = (d.m_pad + 15) / 16;
      P->code_bytes += (int64_t)d.n_stages * d.m_pad * (d.n_pad / 8) * 2;
    }
    P->flops += 2ll * d.batch * d.m_pad * d.n_pad;
    P->max_batch = std::max(P->max_batch, d.batch);
  }

  // ---- per segment: group prefix, range length per warp, grid
  P->gemm_items.clear();
  P->n_tickets = 0;
  for (Segment& s : P->segs) {
    if (!s.tn && s.nb == 1 && fused_enabled() && fused_available(s)) {
      // single-launch form: every layer of the segment reads the same input, at most 8 tokens, and the
      // activations plus the transform scratch fit in shared memory
      const GlqbLinearDesc& d0 = P->descs[P->order[s.first]];
      const bool e8 = s.format == GLQB_FMT_E8_SHELL;
      bool ok = !d0.x_is_rotated && d0.batch <= FUSED_MAX_TOKENS && s.count <= FUSED_MAX_LAYERS;
      {
        // The single-launch form is built for latency: strip-sized work units with a CTA-wide reduction each.  Large
        // launches are bound by streaming instead and keep the three-launch form (E8: with the resident table).
        static const long long max_bytes_trellis = [] { const char* e = getenv("GLQB_FUSED_MAX_BYTES"); return e ? atoll(e) : (1ll << 40); }();
        static const long long max_bytes_e8 = [] { const char* e = getenv("GLQB_FUSED_MAX_BYTES_E8"); return e ? atoll(e) : (16ll << 20); }();
        long long bytes = 0;
        for (int i = 0; i < s.count; ++i) bytes += layer_code_bytes(P->descs[P->order[s.first + i]]);
        ok = ok && bytes <= (e8 ? max_bytes_e8 : max_bytes_trellis);
      }
      for (int i = 1; i < s.count && ok; ++i) ok = same_input(d0, P->descs[P->order[s.first + i]]);
      if (!e8) ok = ok && d0.in_features == d0.n_pad;   // (trellis layers are never padded; the kernel's loads rely on it)
      if (e8) {
        // E8 strips are 16 rows: every output block must hold whole strips; the in-kernel input transform takes
        // blocks of 32 values or more
        for (int i = 0; i < s.count && ok; ++i) {
          const GlqbLinearDesc& d = P->descs[P->order[s.first + i]];
          for (int b = 0; b < d.n_blocks_m; ++b) ok = ok && d.blocks_m[b] >= 16;
        }
        for (int b = 0; b < d0.n_blocks_n; ++b) ok = ok && d0.blocks_n[b] >= 32;
      }
      // wide inputs are transformed once by rht_in_kernel (every CTA recomputing them would cost more than
      // the extra launch); so is a fused RMSNorm whose output block is too long for the in-kernel transform
      static const int in_max_n = [] { const char* e = getenv("GLQB_FUSED_IN_MAX_N"); return e ? atoi(e) : 4096; }();
      bool xr_global = d0.n_pad > in_max_n;
      // Output blocks of at least 2^out_split_log rows are left to rht_out_kernel (S CTAs share one); shorter
      // ones are transformed inside the decode kernel by the CTA that completes them.  Measured on B200 (decoder
      // chain, SmolLM3-3B shapes): an extra launch costs more than the 8192-row transform it takes out of the
      // kernel's tail (101 vs 90 us per layer), so only blocks beyond 8192 rows are split off.
      static const int out_split_log = [] {
        const char* e = getenv("GLQB_FUSED_OUT_SPLIT_LOG");
        return std::max(RHT_SPLIT_MIN_LOG, std::min(e ? atoi(e) : FUSED_OUT_MAX_LOG + 1, FUSED_OUT_MAX_LOG + 1));
      }();
      static const int cta_factor = [] { const char* e = getenv("GLQB_FUSED_CTA_FACTOR"); return e ? std::max(1, atoi(e)) : 1; }();
      int scratch = 32;
      for (int i = 0; i < s.count && ok; ++i) {
        const GlqbLinearDesc& d = P->descs[P->order[s.first + i]];
        for (int b = 0; b < d.n_blocks_m; ++b)           // longer output blocks are left to rht_out_kernel
          if (d.blocks_m[b] < (1 << out_split_log)) scratch = std::max(scratch, d.blocks_m[b]);
      }
      if (!xr_global)
        for (int i = 0; i < d0.n_blocks_n; ++i) scratch = std::max(scratch, d0.blocks_n[i]);
      size_t smem = fused_smem_bytes(d0.n_pad, d0.batch, scratch, e8);
      size_t smem_limit = FUSED_SMEM_LIMIT;
      s.res_entries = 0;
      if (ok && e8 && smem <= FUSED_SMEM_LIMIT) {
        // E8 launches of a few MB and more keep as much of the codebook in shared memory as fits beside the
        // activations (one CTA per SM): otherwise every SM pulls most of the table through L2, one 32-byte sector
        // per gather
        const char* res_env = getenv("GLQB_E8_FUSED_RES_MIN_BYTES");          // (read per plan: the tests switch it)
        const long long res_min = res_env ? atoll(res_env) : (3ll << 20);
        long long bytes = 0;
        const uint32_t* big = nullptr;
        const uint32_t* small = nullptr;
        int small_n = 0;
        if (e8_uniform_tables(P->dev, s, &big, &small, &small_n, &bytes) && bytes >= res_min) {
          const size_t room = FUSED_SMEM_MAX > smem + 1024 ? FUSED_SMEM_MAX - smem - 1024 : 0;
          const int res = (int)std::min<size_t>(65536, room / 4 / 1024 * 1024);
          if (res >= 32768) {
            s.res_entries = res;
            s.big_table = big;
            s.small_table = small ? small : big;
            s.small_entries = small_n;
            smem += (size_t)res * 4 + 1024;
            smem_limit = FUSED_SMEM_MAX;
          }
        }
      }
      if (ok && smem <= smem_limit) {
        int resident = 0;
        CUDA_TRY(fused_prepare(s, smem_limit, smem, &resident));
        if (resident > 0) {
          // column groups per warp and unit: fewer for small layers, so that every SM gets work
          auto units_for = [&](int gpw) {
            long long u = 0;
            for (int i = 0; i < s.count; ++i) {
              const DevLinear& L = P->dev[s.first + i];
              u += (long long)L.strips * ((L.groups_per_strip + MV_WARPS * gpw - 1) / (MV_WARPS * gpw));
            }
            return u;
          };
          // (every CTA repeats the input transform, so more CTAs than SMs only pays when there is more
          // streaming work than one CTA per SM can take)
          // (an E8 group is 256 columns, a trellis group 32.)  No more groups per warp than keep all 8 warps of a
          // unit busy on the narrowest layer: a 4096-wide E8 layer has 16 groups per strip, two per warp.
          int gps_min = 1 << 30;
          for (int i = 0; i < s.count; ++i) gps_min = std::min(gps_min, P->dev[s.first + i].groups_per_strip);
          int gpw = std::min(e8 ? E8F_MAX_GPW : 8, std::max(1, (gps_min + MV_WARPS - 1) / MV_WARPS));
          while (gpw > (e8 ? 1 : 2) && units_for(gpw) < (long long)cta_factor * P->sm_count) gpw >>= 1;
          long long units = units_for(gpw);
          if (units < (1ll << 30)) {
            units = 0;
            for (int i = 0; i < s.count; ++i) {
              DevLinear& L = P->dev[s.first + i];
              const int kch = (L.groups_per_strip + MV_WARPS * gpw - 1) / (MV_WARPS * gpw);
              L.group_base = units;                       // first work unit of the layer
              L.fixed_slots = kch;
              L.slots = kch;
              L.per_warp = gpw;
              L.xr_global = xr_global ? 1 : 0;
              L.out_split_log = out_split_log;
              L.ticket_base = P->n_tickets;
              P->n_tickets += L.nbm;
              units += (long long)L.strips * kch;
            }
            s.fused = true;
            s.total_units = (int)units;
            s.scratch_elems = scratch;
            s.fused_smem = smem;
            s.grid = (int)std::min<long long>(units, (long long)P->sm_count * std::min(resident, 2));
            s.total_groups = 0;
            s.per_warp = 1;
            continue;
          }
        }
      }
    }
    if (s.tn) {
      // tensor-core GEMM: work items = (layer, 128-row tile, token tile[, K split]); the K range is
      // split only when there are too few tiles to occupy the SMs
      long long tiles = 0;
      for (int i = 0; i < s.count; ++i) {
        const DevLinear& L = P->dev[s.first + i];
        tiles += (long long)((L.m + GM_TILE_M - 1) / GM_TILE_M) * ((L.batch + s.tn - 1) / s.tn);
      }
      s.item_first = (int)P->gemm_items.size();
      for (int i = 0; i < s.count; ++i) {
        DevLinear& L = P->dev[s.first + i];
        const int m_tiles = (L.m + GM_TILE_M - 1) / GM_TILE_M, n_tiles = (L.batch + s.tn - 1) / s.tn;
        const int kchunks = (L.n + GM_TILE_K - 1) / GM_TILE_K;
        int ks = 1;
        if (tiles < P->sm_count) ks = (int)std::min<long long>(std::max(1, kchunks / 8), (P->sm_count + tiles - 1) / tiles);
        ks = std::max(1, std::min(ks, 16));
        const int per = (kchunks + ks - 1) / ks;
        ks = (kchunks + per - 1) / per;
        L.fixed_slots = ks;
        L.slots = ks;
        L.gemm_tn = s.tn;
        L.per_warp = 1;
        L.atile_off = s.two_phase ? -1 : 0;      // -1: allocate below
        for (int mt = 0; mt < m_tiles; ++mt)
          for (int nt = 0; nt < n_tiles; ++nt)
            for (int k = 0; k < ks; ++k)
              P->gemm_items.push_back(GemmItem{s.first + i, mt, nt, k * per, std::min(kchunks, (k + 1) * per), k});
        P->max_batch_gemm = std::max(P->max_batch_gemm, L.batch);
      }
      s.item_count = (int)P->gemm_items.size() - s.item_first;
      s.grid = std::min(s.item_count, P->sm_count);
      s.total_groups = 0;
      s.per_warp = 1;
      CUDA_TRY(gemm_prepare(s));
      if (s.two_phase) {
        // tile decode with the codebook resident in shared memory, under the same conditions as the
        // streaming kernel's resident form
        long long bytes = 0;
        const uint32_t* big = nullptr;
        const uint32_t* small = nullptr;
        int small_n = 0;
        if (e8_uniform_tables(P->dev, s, &big, &small, &small_n, &bytes) && bytes >= e8_smem_min_bytes() &&
            tiles_smem_prepare(s.ns) == cudaSuccess) {
          s.smem_table = true;
          s.big_table = big;
          s.small_table = small ? small : big;
          s.small_entries = small_n;
        } else {
          cudaGetLastError();
        }
      }
      continue;
    }
    MvKernel kern = pick_kernel(s);
    int ctas_per_sm = 1;
    CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctas_per_sm, kern, MV_THREADS, 0));
    ctas_per_sm = std::max(1, std::min(ctas_per_sm, 4));
    long long warps_avail = (long long)P->sm_count * ctas_per_sm * MV_WARPS;
    int warps_per_cta = MV_WARPS;
    // E8: keep the codebook in shared memory when the launch is large enough to pay
    // for filling it and every stage reads either one shared 65,536-entry table or one small table
    if (s.format == GLQB_FMT_E8_SHELL && s.nb <= GLQB_E8_SMEM_MAX_NB && pick_e8_smem_kernel(s)) {
      long long bytes = 0;
      const uint32_t* big = nullptr;
      const uint32_t* small = nullptr;
      int small_n = 0;
      const bool ok = e8_uniform_tables(P->dev, s, &big, &small, &small_n, &bytes);
      if (ok && big && bytes >= e8_smem_min_bytes()) {
        E8SmemKernel ck = pick_e8_smem_kernel(s);
        CUDA_TRY(cudaFuncSetAttribute(ck, cudaFuncAttributeMaxDynamicSharedMemorySize, E8S_SMEM_BYTES));
        int resident = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, ck, E8S_THREADS, E8S_SMEM_BYTES) == cudaSuccess &&
            resident > 0) {
          s.smem_table = true;
          s.big_table = big;
          s.small_table = small ? small : big;
          s.small_entries = small_n;
          warps_per_cta = E8S_THREADS / 32;
          warps_avail = (long long)P->sm_count * warps_per_cta;
        } else {
          cudaGetLastError();
        }
      }
    }
    if (s.format == GLQB_FMT_TRELLIS_3INST && s.nb == 1 && s.k2 == 0 && trellis_lut_kernel(s.k1)) {
      long long bytes = 0;
      for (int i = 0; i < s.count; ++i) bytes += (long long)P->dev[s.first + i].m * P->dev[s.first + i].n * s.k1 / 8;
      if (bytes >= trellis_lut_min_bytes() &&
          cudaFuncSetAttribute(trellis_lut_kernel(s.k1), cudaFuncAttributeMaxDynamicSharedMemorySize, MV_LUT_SMEM_BYTES) == cudaSuccess) {
        s.lut_table = true;
        warps_per_cta = MV_LUT_THREADS / 32;
        warps_avail = (long long)P->sm_count * warps_per_cta;
      } else {
        cudaGetLastError();
      }
    }
    long long total = 0;
    for (int i = 0; i < s.count; ++i) {
      DevLinear& L = P->dev[s.first + i];
      L.group_base = total;
      total += (long long)L.strips * L.groups_per_strip;
    }
    s.total_groups = total;
    const long long warps = warps_avail;
    long long per_warp = (total + warps - 1) / warps;
    if (per_warp < 1) per_warp = 1;
    s.per_warp = (int)per_warp;
    const long long used_warps = (total + per_warp - 1) / per_warp;
    s.grid = (int)((used_warps + warps_per_cta - 1) / warps_per_cta);
    for (int i = 0; i < s.count; ++i) {
      DevLinear& L = P->dev[s.first + i];
      L.per_warp = s.per_warp;
      L.slots = (L.groups_per_strip - 1) / s.per_warp + 2;
    }
  }

  // ---- workspace: rotated activations (shared by layers with the same input) + partial sums
  size_t ws = 0;
  P->items_in.clear();
  P->items_in_gemm.clear();
  P->items_out.clear();
  std::vector<char> layer_fused(n, 0);
  for (const Segment& s : P->segs)
    if (s.fused)
      for (int i = 0; i < s.count; ++i) layer_fused[s.first + i] = 1;
  for (int pos = 0; pos < n; ++pos) {
    const GlqbLinearDesc& d = P->descs[P->order[pos]];
    // outside the single-launch form the input transform kernel applies the norm / activation (one token per
    // tile row, at most 8) and the output transform kernel the residual add: decode-sized layers only
    if (!layer_fused[pos] && (d.in_norm_weight || d.in_gated_act || d.y_accumulate) &&
        (d.batch > FUSED_MAX_TOKENS || P->dev[pos].gemm_tn))
      return fail(GLQB_E_INVALID,
                  "layer %d: the fused norm / activation / residual steps are served by the single-launch decode form only "
                  "(at most %d tokens, all layers of the call reading one input)", P->order[pos], FUSED_MAX_TOKENS);
  }
  // a call of a few layers is bound by the latency of one transform item, a sweep of many by their throughput
  const bool latency = n <= FUSED_MAX_LAYERS;
  for (int pos = 0; pos < n; ++pos) {
    DevLinear& L = P->dev[pos];
    const GlqbLinearDesc& d = P->descs[P->order[pos]];
    if (layer_fused[pos]) {                 // activations live in shared memory, transforms run inside the kernel
      ws = align_up(ws, 1024);
      L.xr_off = 0;
      if (L.xr_global) {                    // ... except wide inputs: transformed once into the workspace
        int first = pos;
        while (first > 0 && layer_fused[first - 1] && P->dev[first - 1].xr_global &&
               same_input(P->descs[P->order[first - 1]], d)) --first;
        if (first == pos) {
          L.xr_off = (long long)ws;
          ws = align_up(ws + (size_t)L.batch * L.n * sizeof(__half) * XR_TRELLIS_EXPAND, 1024);
          add_rht_items(P->items_in, pos, L.nbn, L.bn_log, L.batch, P->max_elems_in, latency);
        } else {
          L.xr_off = P->dev[first].xr_off;
        }
      }
      L.part_off = (long long)ws;
      ws = align_up(ws + (size_t)L.slots * L.batch * L.m * sizeof(float), 256);
      L.rstd_off = (long long)ws;
      ws += 256;
      add_rht_items(P->items_out, pos, L.nbm, L.bm_log, L.batch, P->max_elems_out, latency, L.stop_at_yrht ? 64 : L.out_split_log);
      continue;
    }
    int same = -1;
    for (int q = 0; q < pos && same < 0; ++q) {
      if (layer_fused[q]) continue;
      const DevLinear& Q = P->dev[q];
      const GlqbLinearDesc& e = P->descs[P->order[q]];
      if (Q.format == L.format && Q.gemm_tn == L.gemm_tn && Q.n == L.n && Q.in_f == L.in_f && Q.sv == L.sv &&
          Q.batch == L.batch &&
          Q.x_off == L.x_off && Q.x_stride == L.x_stride && Q.x_dtype == L.x_dtype && Q.nbn == L.nbn &&
          Q.x_is_rotated == L.x_is_rotated && Q.in_norm_w == L.in_norm_w && Q.in_norm_dtype == L.in_norm_dtype &&
          Q.in_norm_eps == L.in_norm_eps && Q.in_gated_act == L.in_gated_act &&
          memcmp(e.blocks_n, d.blocks_n, sizeof(int32_t) * d.n_blocks_n) == 0)
        same = q;
    }
    L.xr_global = 1;       // (three-launch form: a fused RMSNorm is complete in the transformed activations)
    if (same >= 0) {
      L.xr_off = P->dev[same].xr_off;
    } else {
      ws = align_up(ws, 1024);
      L.xr_off = (long long)ws;
      if (L.gemm_tn) {
        const size_t n_tiles = (L.batch + L.gemm_tn - 1) / L.gemm_tn, kchunks = (L.n + GM_TILE_K - 1) / GM_TILE_K;
        ws = align_up(ws + n_tiles * kchunks * L.gemm_tn * 128, 256);
        add_rht_items(P->items_in_gemm, pos, L.nbn, L.bn_log, L.batch, P->max_elems_in, false);
      } else {
        // E8 with several tokens interleaves groups of 8 tokens: round the token count up
        const size_t xr_tokens = (L.format == GLQB_FMT_E8_SHELL && L.batch > 1) ? (size_t)((L.batch + 7) / 8 * 8) : (size_t)L.batch;
        ws = align_up(ws + xr_tokens * L.n * sizeof(__half) *
                               (L.format == GLQB_FMT_TRELLIS_3INST ? XR_TRELLIS_EXPAND : 1), 256);
        add_rht_items(P->items_in, pos, L.nbn, L.bn_log, L.batch, P->max_elems_in, latency);
      }
    }
    L.part_off = (long long)ws;
    ws = align_up(ws + (size_t)L.slots * L.batch * L.m * sizeof(float), 256);
    if (L.atile_off < 0) {
      ws = align_up(ws, 1024);
      L.atile_off = (long long)ws;
      ws += (size_t)((L.m + GM_TILE_M - 1) / GM_TILE_M) * ((L.n + GM_TILE_K - 1) / GM_TILE_K) * GM_A_BYTES;
    }
    add_rht_items(P->items_out, pos, L.nbm, L.bm_log, L.batch, P->max_elems_out, latency);
  }
  P->ws_bytes = ws;

  // ---- upload
  CUDA_TRY(cudaMalloc(&P->d_layers, sizeof(DevLinear) * n));
  CUDA_TRY(cudaMemcpy(P->d_layers, P->dev.data(), sizeof(DevLinear) * n, cudaMemcpyHostToDevice));
  CUDA_TRY(cudaMalloc(&P->d_items_in, sizeof(RhtItem) * std::max<size_t>(1, P->items_in.size())));
  CUDA_TRY(cudaMemcpy(P->d_items_in, P->items_in.data(), sizeof(RhtItem) * P->items_in.size(), cudaMemcpyHostToDevice));
  CUDA_TRY(cudaMalloc(&P->d_items_in_gemm, sizeof(RhtItem) * std::max<size_t>(1, P->items_in_gemm.size())));
  CUDA_TRY(cudaMemcpy(P->d_items_in_gemm, P->items_in_gemm.data(), sizeof(RhtItem) * P->items_in_gemm.size(),
                      cudaMemcpyHostToDevice));
  CUDA_TRY(cudaMalloc(&P->d_gemm_items, sizeof(GemmItem) * std::max<size_t>(1, P->gemm_items.size())));
  CUDA_TRY(cudaMemcpy(P->d_gemm_items, P->gemm_items.data(), sizeof(GemmItem) * P->gemm_items.size(),
                      cudaMemcpyHostToDevice));
  CUDA_TRY(cudaMalloc(&P->d_status, sizeof(int)));
  CUDA_TRY(cudaMemset(P->d_status, 0, sizeof(int)));
  CUDA_TRY(cudaMalloc(&P->d_tickets, sizeof(int) * std::max(1, P->n_tickets)));
  CUDA_TRY(cudaMemset(P->d_tickets, 0, sizeof(int) * std::max(1, P->n_tickets)));
  CUDA_TRY(cudaMalloc(&P->d_items_out, sizeof(RhtItem) * std::max<size_t>(1, P->items_out.size())));
  CUDA_TRY(cudaMemcpy(P->d_items_out, P->items_out.data(), sizeof(RhtItem) * P->items_out.size(), cudaMemcpyHostToDevice));

  // The shared-memory limit is a property of the kernel, not of a plan: every plan sets it to the largest
  // value any plan can need (one 32768-value Hadamard block), so a later plan never lowers what an earlier
  // one relies on.
  CUDA_TRY(raise_rht_smem_limits());
  return GLQB_OK;
}


}  // namespace glqb

// =============================================================================================
// exported C ABI
// =============================================================================================
extern "C" {

const char* glqb_last_error(void) { return g_err.c_str(); }
const char* glqb_version(void) { return "glq_b200 0.1 (sm_100a)"; }

int glqb_trellis_kernel_supported(int32_t m, int32_t n) { return (m > 0 && n > 0 && m % 32 == 0 && n % 32 == 0) ? 1 : 0; }

int glqb_plan_create(const GlqbLinearDesc* descs, int32_t count, GlqbPlan** out_plan) {
  if (!descs || count < 1 || !out_plan) return fail(GLQB_E_INVALID, "plan_create: bad arguments");
  for (int i = 0; i < count; ++i) {
    int rc = validate(descs[i], i);
    if (rc) return rc;
  }
  GlqbPlan* P = new GlqbPlan();
  P->descs.assign(descs, descs + count);
  int rc = build_plan(P);
  if (rc) {
    glqb_plan_destroy(P);
    return rc;
  }
  *out_plan = P;
  return GLQB_OK;
}

size_t glqb_plan_workspace_bytes(const GlqbPlan* plan) { return plan ? plan->ws_bytes : 0; }
int64_t glqb_plan_code_bytes(const GlqbPlan* plan) { return plan ? plan->code_bytes : 0; }
int64_t glqb_plan_flops(const GlqbPlan* plan) { return plan ? plan->flops : 0; }
int32_t glqb_plan_launches(const GlqbPlan* plan) {
  if (!plan) return 0;
  int n = (plan->items_in.empty() ? 0 : 1) + (plan->items_in_gemm.empty() ? 0 : 1) + (int)plan->segs.size() +
          (plan->items_out.empty() ? 0 : 1);
  for (const Segment& s : plan->segs) n += s.two_phase;
  return n;
}

int glqb_plan_set_timing(GlqbPlan* plan, int32_t enable) {
  if (!plan) return fail(GLQB_E_INVALID, "null plan");
  plan->timing = enable != 0;
  plan->ev_used = 0;
  return GLQB_OK;
}

int glqb_plan_kernel_ms(GlqbPlan* plan, double* total_ms_out, int32_t* runs_out) {
  if (!plan || !total_ms_out || !runs_out) return fail(GLQB_E_INVALID, "null argument");
  double total = 0.0;
  for (size_t i = 0; i + 1 < plan->ev_used; i += 2) {
    float ms = 0.f;
    CUDA_TRY(cudaEventSynchronize(plan->ev[i + 1]));
    CUDA_TRY(cudaEventElapsedTime(&ms, plan->ev[i], plan->ev[i + 1]));
    total += ms;
  }
  *total_ms_out = total;
  *runs_out = (int32_t)(plan->ev_used / 2);
  return GLQB_OK;
}

int glqb_plan_run(GlqbPlan* P, const void* x_base, void* y_base, void* workspace, size_t workspace_bytes,
                  void* stream_) {
  if (!P || !x_base || !y_base) return fail(GLQB_E_INVALID, "plan_run: null argument");
  if (P->ws_bytes && (!workspace || workspace_bytes < P->ws_bytes))
    return fail(GLQB_E_WORKSPACE, "workspace of %zu bytes needed, %zu given", P->ws_bytes, workspace_bytes);
  if (reinterpret_cast<uintptr_t>(workspace) & 255)
    return fail(GLQB_E_WORKSPACE, "workspace must be 256-byte aligned");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  uint8_t* ws = reinterpret_cast<uint8_t*>(workspace);
  if (!P->items_in.empty()) {
    rht_in_kernel<false><<<(unsigned)P->items_in.size(), rht_threads(P->max_elems_in, P->max_batch), rht_smem(P->max_elems_in), stream>>>(
        P->d_layers, P->d_items_in, reinterpret_cast<const uint8_t*>(x_base), ws);
  }
  if (!P->items_in_gemm.empty()) {
    rht_in_gemm_kernel<<<(unsigned)P->items_in_gemm.size(), rht_threads(P->max_elems_in), rht_smem(P->max_elems_in), stream>>>(
        P->d_layers, P->d_items_in_gemm, reinterpret_cast<const uint8_t*>(x_base), ws);
  }
  if (P->timing) {
    while (P->ev.size() < P->ev_used + 2) {
      cudaEvent_t e;
      CUDA_TRY(cudaEventCreate(&e));
      P->ev.push_back(e);
    }
    CUDA_TRY(cudaEventRecord(P->ev[P->ev_used], stream));
  }
  for (const Segment& s : P->segs) {
    if (s.fused) {
      fused_launch(s, P->dev.data() + s.first, reinterpret_cast<const uint8_t*>(x_base), reinterpret_cast<uint8_t*>(y_base),
                   ws, P->d_tickets, P->comm ? comm_dev(P->comm) : nullptr, stream);
    } else if (s.tn) {
      gemm_launch(s, P->d_layers, P->d_gemm_items + s.item_first, ws, P->d_status, P->sm_count, stream);
    } else if (s.smem_table) {
      pick_e8_smem_kernel(s)<<<s.grid, E8S_THREADS, E8S_SMEM_BYTES, stream>>>(
          P->d_layers + s.first, s.count, s.total_groups, s.per_warp, ws, s.big_table, s.small_table, s.small_entries);
    } else {
      MvKernel kern = pick_kernel(s);
      if (s.lut_table)
        trellis_lut_kernel(s.k1)<<<s.grid, MV_LUT_THREADS, MV_LUT_SMEM_BYTES, stream>>>(P->d_layers + s.first, s.count,
                                                                                       s.total_groups, s.per_warp, ws);
      else
        kern<<<s.grid, MV_THREADS, 0, stream>>>(P->d_layers + s.first, s.count, s.total_groups, s.per_warp, ws);
    }
  }
  if (P->timing) {
    CUDA_TRY(cudaEventRecord(P->ev[P->ev_used + 1], stream));
    P->ev_used += 2;
  }
  if (!P->items_out.empty()) {
    // with programmatic stream serialization: behind the single-launch decode kernel its launch overlaps that
    // kernel's tail (it waits for it before reading anything)
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)P->items_out.size());
    cfg.blockDim = dim3(rht_threads(P->max_elems_out, P->max_batch));
    cfg.dynamicSmemBytes = rht_smem(P->max_elems_out);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const DevLinear* dl = P->d_layers;
    const RhtItem* di = P->d_items_out;
    const uint8_t* cws = ws;
    uint8_t* yb = reinterpret_cast<uint8_t*>(y_base);
    const float* none = nullptr;
    CUDA_TRY(cudaLaunchKernelEx(&cfg, rht_out_kernel<false>, dl, di, cws, yb, none));
  }
  CUDA_TRY(cudaGetLastError());
  return GLQB_OK;
}

int glqb_plan_set_comm(GlqbPlan* P, GlqbComm* comm) {
  if (!P) return fail(GLQB_E_INVALID, "plan_set_comm: null plan");
  if (!comm) {
    for (DevLinear& L : P->dev) L.reduce = 0;
    P->comm = nullptr;
    return GLQB_OK;
  }
  const CommDev* C = comm_dev(comm);
  if (!C) return fail(GLQB_E_INVALID, "plan_set_comm: the communicator is not connected");
  // the sum runs where one CTA holds a whole output block: the single-launch form with every block inside the kernel
  if (!P->items_out.empty()) return fail(GLQB_E_INVALID, "plan_set_comm: the plan transforms outputs in a kernel of its own");
  long long floats = 0;
  int units = 0;
  for (const Segment& s : P->segs) {
    if (!s.fused)
      return fail(GLQB_E_INVALID, "plan_set_comm: only the single-launch decode form (trellis, at most %d tokens) sums over ranks",
                  FUSED_MAX_TOKENS);
    for (int i = s.first; i < s.first + s.count; ++i) {
      DevLinear& L = P->dev[i];
      if (L.stop_at_yrht) return fail(GLQB_E_INVALID, "plan_set_comm: layers that stop before the output transform have no sum");
      L.comm_off = (int)floats;
      L.comm_unit_base = units;
      floats += (long long)L.m * L.batch;
      units += L.nbm;
    }
    // every launch restarts at piece 0: launches of one stream follow one another, and areas alternate by epoch
    if (floats > C->max_floats || units > COMM_MAX_UNITS)
      return fail(GLQB_E_INVALID, "plan_set_comm: a launch exchanges %lld floats in %d pieces; the communicator holds %d and %d",
                  floats, units, C->max_floats, COMM_MAX_UNITS);
    floats = 0;
    units = 0;
  }
  for (DevLinear& L : P->dev) L.reduce = 1;
  P->comm = comm;
  return GLQB_OK;
}

int glqb_plan_status(GlqbPlan* plan, int32_t* status_out) {
  if (!plan || !status_out) return fail(GLQB_E_INVALID, "null argument");
  int v = 0;
  CUDA_TRY(cudaMemcpy(&v, plan->d_status, sizeof(int), cudaMemcpyDeviceToHost));
  *status_out = v;
  if (v) return fail(GLQB_E_DEVICE, "a kernel gave up waiting (status %d): results of that run are invalid", v);
  return GLQB_OK;
}

void glqb_plan_destroy(GlqbPlan* plan) {
  if (!plan) return;
  if (plan->d_layers) cudaFree(plan->d_layers);
  if (plan->d_items_in) cudaFree(plan->d_items_in);
  if (plan->d_items_out) cudaFree(plan->d_items_out);
  if (plan->d_items_in_gemm) cudaFree(plan->d_items_in_gemm);
  if (plan->d_gemm_items) cudaFree(plan->d_gemm_items);
  if (plan->d_status) cudaFree(plan->d_status);
  if (plan->d_tickets) cudaFree(plan->d_tickets);
  for (cudaEvent_t e : plan->ev) cudaEventDestroy(e);
  delete plan;
}

int glqb_decompress_trellis_3inst(const void* packed, int32_t bits, const void* packed2, int32_t bits2,
                                  float inv_resid_scale2, int32_t m, int32_t n, void* out, int32_t out_dtype,
                                  void* stream_) {
  if (!packed || !out || m <= 0 || n <= 0 || m % 32 || n % 32)
    return fail(GLQB_E_INVALID, "decompress_trellis_3inst: needs m %% 32 == 0 and n %% 32 == 0 (got %d x %d)", m, n);
  if (bits < 1 || bits > 4) return fail(GLQB_E_INVALID, "decompress_trellis_3inst: K=%d unsupported (1..4)", bits);
  const int k2 = packed2 ? bits2 : 0;
  if (packed2 && (bits2 < 1 || bits2 > 4)) return fail(GLQB_E_INVALID, "decompress_trellis_3inst: K2=%d", bits2);
  if (out_dtype != GLQB_DT_F16 && out_dtype != GLQB_DT_F32) return fail(GLQB_E_INVALID, "out dtype");
  if (k2 && out_dtype != GLQB_DT_F32) return fail(GLQB_E_INVALID, "two-stage decode is written as fp32");
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  const long long groups = (long long)(m / 32) * (n / 32);
  const int grid = (int)std::min<long long>((groups + MV_WARPS - 1) / MV_WARPS, 148 * 8);
  const uint8_t* p1 = reinterpret_cast<const uint8_t*>(packed);
  const uint8_t* p2 = reinterpret_cast<const uint8_t*>(packed2);
  const int f32 = out_dtype == GLQB_DT_F32;
#define D_CASE(A, B)                                                                                      \
  if (bits == A && k2 == B) {                                                                             \
    trellis_dump_kernel<A, B><<<grid, MV_THREADS, 0, stream>>>(p1, p2, inv_resid_scale2, m, n, out, f32); \
    CUDA_TRY(cudaGetLastError());                                                                         \
    return GLQB_OK;                                                                                       \
  }
#ifdef GLQB_FAST_BUILD   /* developer builds for kernel experiments: the 4-bit single-stage rate only */
  D_CASE(4, 0)
#else
  D_CASE(1, 0) D_CASE(2, 0) D_CASE(3, 0) D_CASE(4, 0)
  D_CASE(4, 1) D_CASE(4, 2) D_CASE(4, 3) D_CASE(4, 4)
#endif
#undef D_CASE
  return fail(GLQB_E_INVALID, "decompress_trellis_3inst: no kernel for K=%d+%d", bits, k2);
}

int glqb_dequant_e8(const void* const* qidxs, const uint32_t* const* tables, const int32_t* table_entries,
                    const float* stage_scale, int32_t n_stages, int32_t m, int32_t n, float* out, void* stream_) {
  if (!qidxs || !tables || !table_entries || !out || n_stages < 1 || n_stages > 4 || m <= 0 || n <= 0 || n % 8)
    return fail(GLQB_E_INVALID, "dequant_e8: bad arguments");
  E8DumpArgs A;
  memset(&A, 0, sizeof A);
  for (int s = 0; s < n_stages; ++s) {
    if (!qidxs[s] || !tables[s]) return fail(GLQB_E_INVALID, "dequant_e8: stage %d null", s);
    const int e = table_entries[s];
    if (e < 1 || e > 65536 || (e & (e - 1))) return fail(GLQB_E_INVALID, "dequant_e8: table entries %d", e);
    A.q[s] = reinterpret_cast<const uint16_t*>(qidxs[s]);
    A.table[s] = tables[s];
    A.entries[s] = e;
    A.scale[s] = (s && stage_scale) ? stage_scale[s] : 1.0f;
  }
  A.n_stages = n_stages; A.m = m; A.n = n;
  const long long total = (long long)m * (n / 8);
  const int grid = (int)std::min<long long>((total + 255) / 256, 148 * 16);
  e8_dump_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(A, out);
  CUDA_TRY(cudaGetLastError());
  return GLQB_OK;
}

int glqb_e8_pack_table(const void* codebook_f16, int32_t entries, uint32_t* out_packed, void* stream_) {
  if (!codebook_f16 || !out_packed || entries < 1) return fail(GLQB_E_INVALID, "e8_pack_table: bad arguments");
  e8_pack_table_kernel<<<(entries + 255) / 256, 256, 0, reinterpret_cast<cudaStream_t>(stream_)>>>(
      reinterpret_cast<const __half*>(codebook_f16), entries, out_packed);
  CUDA_TRY(cudaGetLastError());
  return GLQB_OK;
}

// The unfused transform ops describe their one layer in kernel-parameter space (rht_in_single_kernel /
// rht_out_single_kernel): no device table, no allocation, no copy, nothing that would be illegal while the
// stream is being captured into a CUDA graph.  `offsets` (optional) gives the first column of every
// Hadamard block; without it the blocks are laid side by side.
static int run_rht_single(bool input, const void* src, int src_dtype, int64_t src_stride, const void* signs,
                          void* dst, int dst_dtype, int64_t dst_stride, int32_t feat, int32_t pad,
                          const int32_t* offsets, const int32_t* blocks, int32_t n_blocks, int32_t batch,
                          cudaStream_t stream) {
  if (!src || !signs || !dst || !blocks || n_blocks < 1 || n_blocks > GLQB_MAX_BLOCKS || batch < 1 || feat < 1 ||
      feat > pad)
    return fail(GLQB_E_INVALID, "rht: bad arguments (at most %d Hadamard blocks per call)", GLQB_MAX_BLOCKS);
  if (reinterpret_cast<uintptr_t>(signs) & 15) return fail(GLQB_E_INVALID, "rht: sign vector must be 16-byte aligned");
  DevLinear L;
  memset(&L, 0, sizeof L);
  RhtSingle S;
  memset(&S, 0, sizeof S);
  int off = 0, max_elems = 32, ctas = 0;
  for (int i = 0; i < n_blocks; ++i) {
    const int b = blocks[i];
    if (b < 1 || (b & (b - 1)) || b > 32768) return fail(GLQB_E_INVALID, "rht: block %d", b);
    const int o = offsets ? offsets[i] : off;
    if (o < 0 || o + b > pad) return fail(GLQB_E_INVALID, "rht: block %d at column %d exceeds %d columns", b, o, pad);
    if (input) { L.bn_off[i] = o; L.bn_log[i] = ilog2(b); } else { L.bm_off[i] = o; L.bm_log[i] = ilog2(b); }
    off += b;
    const int tt = rht_tile_tokens(b, batch);
    S.first_cta[i] = ctas;
    S.tile_tokens[i] = tt;
    ctas += (batch + tt - 1) / tt;
    max_elems = std::max(max_elems, tt * b);
  }
  S.first_cta[n_blocks] = ctas;
  S.n_blocks = n_blocks;
  if (!offsets && off != pad) return fail(GLQB_E_INVALID, "rht: blocks sum to %d, expected %d", off, pad);
  L.format = GLQB_FMT_E8_SHELL;
  L.batch = batch;
  if (input) {
    L.n = pad; L.in_f = feat; L.sv = reinterpret_cast<const __half*>(signs);
    L.x_dtype = src_dtype; L.x_stride = src_stride; L.nbn = n_blocks; L.xr_off = 0;
  } else {
    L.m = pad; L.out_f = feat; L.su = reinterpret_cast<const __half*>(signs);
    L.y_dtype = dst_dtype; L.y_stride = dst_stride; L.nbm = n_blocks; L.wscale = 1.f;
  }
  int dev_id = 0;
  CUDA_TRY(cudaGetDevice(&dev_id));
  {
    // once per device: the two kernels may need more than the default 48 KiB of dynamic shared memory
    static std::mutex mu;
    static bool done[64] = {false};
    std::lock_guard<std::mutex> lock(mu);
    if (dev_id >= 0 && dev_id < 64 && !done[dev_id]) {
      const int lim = rht_smem(32768);
      CUDA_TRY(cudaFuncSetAttribute(rht_in_single_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
      CUDA_TRY(cudaFuncSetAttribute(rht_out_single_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, lim));
      done[dev_id] = true;
    }
  }
  const int smem = rht_smem(max_elems);
  if (input)
    rht_in_single_kernel<<<(unsigned)ctas, rht_threads(max_elems), smem, stream>>>(
        L, S, reinterpret_cast<const uint8_t*>(src), reinterpret_cast<uint8_t*>(dst));
  else
    rht_out_single_kernel<<<(unsigned)ctas, rht_threads(max_elems), smem, stream>>>(
        L, S, reinterpret_cast<uint8_t*>(dst), reinterpret_cast<const float*>(src));
  CUDA_TRY(cudaGetLastError());
  return GLQB_OK;
}

int glqb_input_rht(const void* x, int32_t x_dtype, int64_t x_stride, const void* sv, void* out_f32,
                   int32_t in_features, int32_t n_pad, const int32_t* blocks, int32_t n_blocks, int32_t batch,
                   void* stream) {
  return run_rht_single(true, x, x_dtype, x_stride, sv, out_f32, GLQB_DT_F32, n_pad, in_features, n_pad, nullptr,
                        blocks, n_blocks, batch, reinterpret_cast<cudaStream_t>(stream));
}

int glqb_output_rht(const float* y_rht, const void* su, void* out, int32_t out_dtype, int64_t out_stride,
                    int32_t out_features, int32_t m_pad, const int32_t* blocks, int32_t n_blocks, int32_t batch,
                    void* stream) {
  return run_rht_single(false, y_rht, GLQB_DT_F32, m_pad, su, out, out_dtype, out_stride, out_features, m_pad,
                        nullptr, blocks, n_blocks, batch, reinterpret_cast<cudaStream_t>(stream));
}

int glqb_output_rht_shards(const float* y_rht, const void* su, void* out, int32_t out_dtype, int64_t out_stride,
                           int32_t out_features, int32_t total_m, const int32_t* offsets, const int32_t* blocks,
                           int32_t n_blocks, int32_t batch, void* stream) {
  if (!offsets) return fail(GLQB_E_INVALID, "output_rht_shards: null offsets");
  return run_rht_single(false, y_rht, GLQB_DT_F32, total_m, su, out, out_dtype, out_stride, out_features, total_m,
                        offsets, blocks, n_blocks, batch, reinterpret_cast<cudaStream_t>(stream));
}

size_t glqb_linear_workspace_bytes(const GlqbLinearDesc* desc) {
  // Upper bound that does not depend on the device, with the roundings build_plan applies: activations
  // (E8 batches are padded to 8 tokens; the GEMM path stores whole token tiles of whole 64-column chunks),
  // the largest possible number of partial-sum slots (one per work group of a strip, plus one), and for
  // E8 above 128 tokens the decoded fp16 weight tiles.
  if (!desc) return 0;
  const size_t batch = (size_t)std::max(1, desc->batch);
  const int tn = tn_for_batch((int)batch);
  size_t ws = 1024;
  if (tn) {
    const size_t n_tiles = (batch + tn - 1) / tn, kchunks = ((size_t)desc->n_pad + GM_TILE_K - 1) / GM_TILE_K;
    ws += align_up(n_tiles * kchunks * tn * 128, 1024);
    ws += align_up(16 * batch * desc->m_pad * 4, 1024);                      // at most 16 K splits
    if (desc->format == GLQB_FMT_E8_SHELL)
      ws += align_up((size_t)((desc->m_pad + GM_TILE_M - 1) / GM_TILE_M) * kchunks * GM_A_BYTES, 1024) + 1024;
  } else {
    const size_t gps = desc->format == GLQB_FMT_TRELLIS_3INST ? desc->n_pad / 32 : (desc->n_pad + 255) / 256;
    ws += align_up(((batch + 7) / 8 * 8) * desc->n_pad * 2 * XR_TRELLIS_EXPAND, 1024);
    ws += align_up((gps + 1) * batch * desc->m_pad * 4, 1024);
  }
  return ws;
}

int glqb_fused_linear(const GlqbLinearDesc* desc, const void* x, void* y, void* workspace, size_t workspace_bytes,
                      void* stream) {
  // Stateless convenience form: builds a one-layer plan (which allocates its small device table), runs it,
  // waits for the stream and releases the plan.  It therefore synchronises and must not be called while the
  // stream is being captured; callers on a hot path keep a plan instead (glqb_plan_create once).
  GlqbPlan* P = nullptr;
  int rc = glqb_plan_create(desc, 1, &P);
  if (rc) return rc;
  rc = glqb_plan_run(P, x, y, workspace, workspace_bytes, stream);
  cudaError_t e = cudaStreamSynchronize(reinterpret_cast<cudaStream_t>(stream));
  glqb_plan_destroy(P);
  if (rc) return rc;
  if (e != cudaSuccess) return fail(GLQB_E_CUDA, "fused_linear: %s", cudaGetErrorString(e));
  return GLQB_OK;
}

}  // extern "C"
