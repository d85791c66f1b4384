// glqb_trellis_linear_noalloc — a batch-1 trellis 3INST linear whose scratch memory lives inside the
// library instead of coming from the caller or from an allocator.
//
// Who this is for: code that may not allocate device memory at the point where it has to run a
// layer — for example a plugin called from inside someone else's memory-pool callback, a host that
// pre-sized all of its device memory at start-up and forbids later cudaMalloc calls (real-time or
// safety-certified loops), or a caller that holds no torch allocator at all (a bare C program that
// only links this library).  The ordinary entry points avoid per-call allocation too, but they need
// a caller-provided workspace and a plan whose small device table was allocated when it was built;
// this one needs neither.  It has no counterpart in the reference project.
//
// How: the rotated activations and the per-warp partial sums go to a file-scope __device__ array
// (NA_SCRATCH_BYTES, a few MiB that every GPU which loads the library keeps until the process
// exits); the layer description travels by value in kernel-parameter space.  Nothing in this file
// calls cudaMalloc, cudaFree or any allocating library routine.
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "glqb_kernels.cuh"

namespace glqb {

// Upper bounds of the entry point (stated in include/glq_b200.h).
constexpr int NA_MAX_DIM = 32768;                         // m_pad and n_pad
constexpr size_t NA_SCRATCH_BYTES = 4u << 20;             // 4 MiB per device
constexpr size_t NA_XR_BYTES = (size_t)NA_MAX_DIM * 2 * XR_TRELLIS_EXPAND;   // activations come first

// In device code `g_na_scratch` names the array itself.  In host code the same identifier is only a
// stand-in symbol: its device address has to be asked for with cudaGetSymbolAddress (below).
static __device__ __align__(256) unsigned char g_na_scratch[NA_SCRATCH_BYTES];

static std::mutex g_na_mutex;
static unsigned char* g_na_ptr[64] = {nullptr};   // per device ordinal, filled on first use

static int na_fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  set_error_message(buf);      // read back with glqb_last_error()
  return code;
}

// ---- kernels: same device functions as the ordinary path, layer passed by value ------------------
__global__ void __launch_bounds__(1024) na_rht_in_kernel(const __grid_constant__ DevLinear L,
                                                         const uint8_t* __restrict__ x, uint8_t* __restrict__ ws) {
  extern __shared__ float fbuf[];
  const int blk = blockIdx.x;
  const int off = L.bn_off[blk], logbs = L.bn_log[blk], bs = 1 << logbs;
  for (int i = threadIdx.x; i < bs; i += blockDim.x) {
    const int col = off + i;
    fbuf[i] = load_act(x, col, L.x_dtype) * __half2float(L.sv[col]);
  }
  fht_smem(fbuf, logbs);
  const float rs = rsqrtf((float)bs);
  __half2* out = reinterpret_cast<__half2*>(ws + L.xr_off);
  for (int i = threadIdx.x; i < bs; i += blockDim.x) {
    const int col = off + i;
    const int pos = (col & ~31) * XR_TRELLIS_EXPAND + xr_pos_trellis(col & 31);
    out[pos >> 1] = __halves2half2(__float2half_rn(fbuf[i] * rs), __float2half_rn(0.f));
  }
}

template <int K>
__global__ void __launch_bounds__(MV_THREADS) na_trellis_mv_kernel(const __grid_constant__ DevLinear L,
                                                                   long long total_groups, int per_warp,
                                                                   uint8_t* __restrict__ ws) {
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * MV_WARPS + (threadIdx.x >> 5);
  long long g = w * per_warp;
  const long long gend = min(g + per_warp, total_groups);
  const int gq = lane >> 2, tq = lane & 3;
  const int gps = L.groups_per_strip;
  const __half* xr = reinterpret_cast<const __half*>(ws + L.xr_off);
  while (g < gend) {
    const int strip = (int)(g / gps);
    const int c0 = (int)(g - (long long)strip * gps);
    const int c1 = (int)min((long long)gps, c0 + (gend - g));
    float acc[1][2][4];
#pragma unroll
    for (int mi = 0; mi < 2; ++mi)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[0][mi][i] = 0.f;
    const uint8_t* p = L.codes[0] + ((long long)strip * gps + c0) * (128 * K) + lane * (4 * K);
    const uint4* xq = reinterpret_cast<const uint4*>(xr + (long long)c0 * 32 * XR_TRELLIS_EXPAND + tq * 16);
    for (int c = c0; c < c1; ++c) {
      const Words<K> v = load_words<K>(p);
      uint4 xb[1][2];
      xb[0][0] = xb[0][1] = make_uint4(0u, 0u, 0u, 0u);
      if (gq == 0) { xb[0][0] = __ldg(xq); xb[0][1] = __ldg(xq + 1); }
      group_mma<K, 1>(v, lane, xb, acc);
      p += 128 * K;
      xq += 8;
    }
    const int slot = (int)(w - ((long long)strip * gps) / per_warp);
    float* part = reinterpret_cast<float*>(ws + L.part_off) + (long long)slot * L.m;
    if (tq == 0) {
#pragma unroll
      for (int mi = 0; mi < 2; ++mi) {
        part[strip * 32 + mi * 16 + gq] = acc[0][mi][0];
        part[strip * 32 + mi * 16 + gq + 8] = acc[0][mi][2];
      }
    }
    g += c1 - c0;
  }
}

__global__ void __launch_bounds__(1024) na_rht_out_kernel(const __grid_constant__ DevLinear L,
                                                          const uint8_t* __restrict__ ws, uint8_t* __restrict__ y) {
  extern __shared__ float fbuf[];
  const int blk = blockIdx.x;
  const int off = L.bm_off[blk], logbs = L.bm_log[blk], bs = 1 << logbs;
  for (int i = threadIdx.x; i < bs; i += blockDim.x) {
    const int row = off + i;
    const int strip = row >> 5;
    const long long g0 = (long long)strip * L.groups_per_strip;
    const int cnt = (int)((g0 + L.groups_per_strip - 1) / L.per_warp - g0 / L.per_warp) + 1;
    const float* p = reinterpret_cast<const float*>(ws + L.part_off) + row;
    float s = 0.f;
    for (int k = 0; k < cnt; ++k) s += p[(long long)k * L.m];
    fbuf[i] = s * L.wscale;
  }
  fht_smem(fbuf, logbs);
  const float rs = rsqrtf((float)bs);
  for (int i = threadIdx.x; i < bs; i += blockDim.x) {
    const int row = off + i;
    store_act(y, row, L.y_dtype, fbuf[i] * rs * __half2float(L.su[row]));
  }
}

typedef void (*NaMvKernel)(const DevLinear, long long, int, uint8_t*);

}  // namespace glqb

using namespace glqb;

extern "C" {

size_t glqb_noalloc_scratch_bytes(void) { return NA_SCRATCH_BYTES; }

int glqb_trellis_linear_noalloc(const void* x, int32_t x_dtype, void* y, int32_t y_dtype, const void* packed,
                                int32_t bits, const void* su, const void* sv, float wscale, int32_t m, int32_t n,
                                const int32_t* blocks_n, int32_t n_blocks_n, const int32_t* blocks_m,
                                int32_t n_blocks_m, void* stream_) {
  if (!x || !y || !packed || !su || !sv || !blocks_n || !blocks_m)
    return na_fail(GLQB_E_INVALID, "trellis_linear_noalloc: null argument");
  if (m <= 0 || n <= 0 || m % 32 || n % 32)
    return na_fail(GLQB_E_INVALID, "trellis_linear_noalloc: needs m %% 32 == 0 and n %% 32 == 0 (got %d x %d)", m, n);
  if (m > NA_MAX_DIM || n > NA_MAX_DIM)
    return na_fail(GLQB_E_INVALID,
                   "trellis_linear_noalloc: %d x %d exceeds the built-in scratch (both dimensions must be <= %d); "
                   "use glqb_plan_create / glqb_plan_run with a caller workspace for larger layers",
                   m, n, NA_MAX_DIM);
  if (bits < 1 || bits > 4) return na_fail(GLQB_E_INVALID, "trellis_linear_noalloc: K=%d unsupported (1..4)", bits);
  if (x_dtype < 0 || x_dtype > 2 || y_dtype < 0 || y_dtype > 2)
    return na_fail(GLQB_E_INVALID, "trellis_linear_noalloc: dtype");
  if (n_blocks_n < 1 || n_blocks_n > GLQB_MAX_BLOCKS || n_blocks_m < 1 || n_blocks_m > GLQB_MAX_BLOCKS)
    return na_fail(GLQB_E_INVALID, "trellis_linear_noalloc: block counts");

  DevLinear L;
  memset(&L, 0, sizeof L);
  int off = 0, max_in = 32, max_out = 32;
  for (int i = 0; i < n_blocks_n; ++i) {
    const int b = blocks_n[i];
    if (b < 32 || (b & (b - 1))) return na_fail(GLQB_E_INVALID, "trellis_linear_noalloc: blocks_n[%d]=%d", i, b);
    L.bn_off[i] = off; L.bn_log[i] = 31 - __builtin_clz((unsigned)b); off += b; max_in = std::max(max_in, b);
  }
  if (off != n) return na_fail(GLQB_E_INVALID, "trellis_linear_noalloc: blocks_n sum to %d, expected %d", off, n);
  off = 0;
  for (int i = 0; i < n_blocks_m; ++i) {
    const int b = blocks_m[i];
    if (b < 32 || (b & (b - 1))) return na_fail(GLQB_E_INVALID, "trellis_linear_noalloc: blocks_m[%d]=%d", i, b);
    L.bm_off[i] = off; L.bm_log[i] = 31 - __builtin_clz((unsigned)b); off += b; max_out = std::max(max_out, b);
  }
  if (off != m) return na_fail(GLQB_E_INVALID, "trellis_linear_noalloc: blocks_m sum to %d, expected %d", off, m);

  // ---- once per device: the device address of the scratch array
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return na_fail(GLQB_E_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= 64) return na_fail(GLQB_E_INVALID, "trellis_linear_noalloc: device ordinal %d", dev);
  unsigned char* scratch = nullptr;
  int sm_count = 0;
  {
    std::lock_guard<std::mutex> lock(g_na_mutex);
    if (!g_na_ptr[dev]) {
      // `dev` is the current device here, so the address returned is the copy of the array that
      // lives on this GPU.  Passing the bare symbol to a kernel instead would hand it a host-side
      // placeholder address.
      unsigned char* ptr = nullptr;
      e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_na_scratch);
      if (e != cudaSuccess || !ptr)
        return na_fail(GLQB_E_CUDA, "cudaGetSymbolAddress(g_na_scratch): %s", cudaGetErrorString(e));
      const int smem_in = NA_MAX_DIM * 4;
      e = cudaFuncSetAttribute(na_rht_in_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_in);
      if (e == cudaSuccess)
        e = cudaFuncSetAttribute(na_rht_out_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_in);
      if (e != cudaSuccess) return na_fail(GLQB_E_CUDA, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      g_na_ptr[dev] = ptr;
    }
    scratch = g_na_ptr[dev];
  }
  e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return na_fail(GLQB_E_CUDA, "cudaDeviceGetAttribute: %s", cudaGetErrorString(e));

  L.codes[0] = reinterpret_cast<const uint8_t*>(packed);
  L.su = reinterpret_cast<const __half*>(su);
  L.sv = reinterpret_cast<const __half*>(sv);
  L.wscale = wscale;
  L.format = GLQB_FMT_TRELLIS_3INST;
  L.m = m; L.n = n; L.in_f = n; L.out_f = m; L.n_stages = 1; L.bits[0] = bits;
  L.batch = 1; L.x_dtype = x_dtype; L.y_dtype = y_dtype;
  L.nbn = n_blocks_n; L.nbm = n_blocks_m;
  L.groups_per_strip = n / 32;
  L.strips = m / 32;
  L.xr_off = 0;
  L.part_off = (long long)NA_XR_BYTES;

  // Split the groups over warps; the range handed to each warp is grown, if needed, until the
  // partial sums (slots x m floats) fit behind the activations.
  const long long total = (long long)L.strips * L.groups_per_strip;
  const long long warps = (long long)sm_count * 3 * MV_WARPS;
  long long per_warp = std::max<long long>(1, (total + warps - 1) / warps);
  const size_t part_room = NA_SCRATCH_BYTES - NA_XR_BYTES;
  for (;;) {
    const size_t slots = (size_t)(L.groups_per_strip - 1) / per_warp + 2;
    if (slots * (size_t)m * sizeof(float) <= part_room) break;
    ++per_warp;
  }
  L.per_warp = (int)per_warp;
  L.slots = (L.groups_per_strip - 1) / L.per_warp + 2;
  const long long used_warps = (total + per_warp - 1) / per_warp;
  const int grid = (int)((used_warps + MV_WARPS - 1) / MV_WARPS);

  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  na_rht_in_kernel<<<n_blocks_n, std::max(64, std::min(1024, max_in / 8)), max_in * 4, stream>>>(
      L, reinterpret_cast<const uint8_t*>(x), scratch);
  NaMvKernel kern = bits == 4 ? na_trellis_mv_kernel<4> : bits == 3 ? na_trellis_mv_kernel<3>
                  : bits == 2 ? na_trellis_mv_kernel<2> : na_trellis_mv_kernel<1>;
  kern<<<grid, MV_THREADS, 0, stream>>>(L, total, L.per_warp, scratch);
  na_rht_out_kernel<<<n_blocks_m, std::max(64, std::min(1024, max_out / 8)), max_out * 4, stream>>>(
      L, scratch, reinterpret_cast<uint8_t*>(y));
  e = cudaGetLastError();
  if (e != cudaSuccess) return na_fail(GLQB_E_CUDA, "trellis_linear_noalloc launch: %s", cudaGetErrorString(e));
  return GLQB_OK;
}

}  // extern "C"
