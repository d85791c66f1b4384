// Communicator for the in-kernel sums over tensor-parallel ranks (glqb_comm.cuh): buffer set-up, the mapping of the
// peers' receive areas (CUDA IPC between processes of one node, or plain pointers inside one process), and a
// stand-alone all-reduce of one fp32 buffer.  The reference sums row-parallel partial results with NCCL through its
// host framework (glq_vllm/linear_method.py:1031-1102 runs under vLLM's RowParallelLinear); this replaces that sum
// for decode-sized messages, where launch and protocol latency is the whole cost.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <vector>

#include "glqb_internal.h"
#include "glqb_comm.cuh"
#include "glqb_launch.h"

struct GlqbComm {
  glqb::CommDev dev = {};
  int device = 0;
  unsigned char* base = nullptr;                 // this rank's area (owned)
  size_t bytes = 0;
  void* peer_base[glqb::COMM_MAX_RANKS] = {};    // mapped peers (IPC mappings are closed on destroy)
  bool peer_ipc[glqb::COMM_MAX_RANKS] = {};
  bool connected = false;
};

namespace glqb {

static int comm_fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  set_error_message(buf);
  return code;
}
#define COMM_TRY(expr)                                                                          \
  do {                                                                                          \
    cudaError_t _e = (expr);                                                                    \
    if (_e != cudaSuccess) return comm_fail(GLQB_E_CUDA, "%s: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

static size_t comm_flag_bytes(int world) { return (size_t)2 * world * COMM_MAX_UNITS * sizeof(int); }

static void comm_point(GlqbComm* c, int r, void* base) {
  unsigned char* b = reinterpret_cast<unsigned char*>(base);
  c->peer_base[r] = base;
  c->dev.flags[r] = reinterpret_cast<int*>(b + COMM_CTRL_BYTES);
  c->dev.data[r] = reinterpret_cast<float*>(b + COMM_CTRL_BYTES + comm_flag_bytes(c->dev.world));
}

const CommDev* comm_dev(const GlqbComm* c) { return (c && c->connected) ? &c->dev : nullptr; }

// One CTA per chunk: store the chunk into every rank's area, exchange flags, add the sources up in rank order.
constexpr int AR_THREADS = 256;
constexpr int AR_CHUNK = 2048;                   // floats per CTA: two float4 per thread
static __global__ void __launch_bounds__(AR_THREADS)
comm_all_reduce_kernel(const __grid_constant__ CommDev C, float* __restrict__ buf, int count, int chunk) {
  const int e = comm_epoch(C);
  const int c0 = blockIdx.x * chunk, c1 = min(count, c0 + chunk);
  for (int i = c0 + threadIdx.x * 4; i < c1; i += AR_THREADS * 4) {
    float v[4];
    for (int k = 0; k < 4; ++k) v[k] = (i + k < c1) ? buf[i + k] : 0.f;
    for (int r = 0; r < C.world; ++r) {
      float* dst = comm_slot(C, r, e, C.rank) + i;         // chunk starts are multiples of 4: 16-byte aligned
      *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
    }
  }
  comm_signal_and_wait(C, e, blockIdx.x);
  for (int i = c0 + threadIdx.x * 4; i < c1; i += AR_THREADS * 4) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < C.world; ++r) {
      const float4 t = __ldcg(reinterpret_cast<const float4*>(comm_slot(C, C.rank, e, r) + i));
      s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
    }
    const float o[4] = {s.x, s.y, s.z, s.w};
    for (int k = 0; k < 4; ++k)
      if (i + k < c1) buf[i + k] = o[k];
  }
  comm_cta_done(C, e);
}

}  // namespace glqb

using namespace glqb;

extern "C" {

int glqb_comm_create(int32_t rank, int32_t world, int64_t max_floats, GlqbComm** out) {
  if (!out) return comm_fail(GLQB_E_INVALID, "comm_create: null argument");
  if (world < 1 || world > COMM_MAX_RANKS || rank < 0 || rank >= world)
    return comm_fail(GLQB_E_INVALID, "comm_create: rank %d of %d (at most %d ranks)", rank, world, COMM_MAX_RANKS);
  if (max_floats < 4 || max_floats > (1 << 24) || max_floats % 4)
    return comm_fail(GLQB_E_INVALID, "comm_create: max_floats %lld (a multiple of 4, at most 2^24)", (long long)max_floats);
  GlqbComm* c = new GlqbComm;
  c->dev.rank = rank;
  c->dev.world = world;
  c->dev.max_floats = (int)max_floats;
  c->dev.wait_ns = 2000ll * 1000 * 1000;          // two seconds
  c->bytes = COMM_CTRL_BYTES + comm_flag_bytes(world) + (size_t)2 * world * max_floats * sizeof(float);
  cudaError_t e = cudaGetDevice(&c->device);
  if (e == cudaSuccess) e = cudaMalloc(&c->base, c->bytes);
  if (e == cudaSuccess) e = cudaMemset(c->base, 0, c->bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    if (c->base) cudaFree(c->base);
    delete c;
    return comm_fail(GLQB_E_CUDA, "comm_create: %s", cudaGetErrorString(e));
  }
  c->dev.epoch = reinterpret_cast<int*>(c->base);
  c->dev.done = reinterpret_cast<int*>(c->base) + 1;
  c->dev.status = reinterpret_cast<int*>(c->base) + 2;
  comm_point(c, rank, c->base);
  c->connected = world == 1;
  *out = c;
  return GLQB_OK;
}

int glqb_comm_handle(GlqbComm* c, void* handle_out, int32_t handle_bytes) {
  if (!c || !handle_out) return comm_fail(GLQB_E_INVALID, "comm_handle: null argument");
  if (handle_bytes < (int)sizeof(cudaIpcMemHandle_t))
    return comm_fail(GLQB_E_INVALID, "comm_handle: %d bytes given, %zu needed", handle_bytes, sizeof(cudaIpcMemHandle_t));
  cudaIpcMemHandle_t h;
  COMM_TRY(cudaIpcGetMemHandle(&h, c->base));
  memcpy(handle_out, &h, sizeof(h));
  return GLQB_OK;
}

int glqb_comm_connect(GlqbComm* c, const void* handles, int32_t handle_stride) {
  if (!c || !handles) return comm_fail(GLQB_E_INVALID, "comm_connect: null argument");
  if (handle_stride < (int)sizeof(cudaIpcMemHandle_t)) return comm_fail(GLQB_E_INVALID, "comm_connect: handle stride");
  for (int r = 0; r < c->dev.world; ++r) {
    if (r == c->dev.rank || c->peer_base[r]) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, reinterpret_cast<const unsigned char*>(handles) + (size_t)r * handle_stride, sizeof(h));
    void* p = nullptr;
    COMM_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    c->peer_ipc[r] = true;
    comm_point(c, r, p);
  }
  c->connected = true;
  return GLQB_OK;
}

int glqb_comm_connect_local(GlqbComm* c, GlqbComm* const* comms) {
  if (!c || !comms) return comm_fail(GLQB_E_INVALID, "comm_connect_local: null argument");
  for (int r = 0; r < c->dev.world; ++r) {
    if (r == c->dev.rank) continue;
    const GlqbComm* o = comms[r];
    if (!o || o->dev.world != c->dev.world || o->dev.rank != r || o->dev.max_floats != c->dev.max_floats)
      return comm_fail(GLQB_E_INVALID, "comm_connect_local: entry %d is not rank %d of the same communicator", r, r);
    if (o->device != c->device) {
      int can = 0;
      COMM_TRY(cudaDeviceCanAccessPeer(&can, c->device, o->device));
      if (!can) return comm_fail(GLQB_E_INVALID, "comm_connect_local: device %d cannot map device %d", c->device, o->device);
      cudaError_t e = cudaDeviceEnablePeerAccess(o->device, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled)
        return comm_fail(GLQB_E_CUDA, "cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(e));
      cudaGetLastError();
    }
    comm_point(c, r, o->base);
  }
  c->connected = true;
  return GLQB_OK;
}

int glqb_comm_set_timeout_ms(GlqbComm* c, int32_t ms) {
  if (!c || ms < 1 || ms > 60000) return comm_fail(GLQB_E_INVALID, "comm_set_timeout_ms: 1..60000 ms");
  c->dev.wait_ns = (long long)ms * 1000 * 1000;
  return GLQB_OK;
}

int64_t glqb_comm_max_floats(const GlqbComm* c) { return c ? c->dev.max_floats : 0; }

int glqb_comm_all_reduce(GlqbComm* c, void* buf_f32, int64_t count, void* stream) {
  if (!c || !buf_f32) return comm_fail(GLQB_E_INVALID, "comm_all_reduce: null argument");
  if (!c->connected) return comm_fail(GLQB_E_INVALID, "comm_all_reduce: the communicator is not connected");
  if (count < 1 || count > c->dev.max_floats)
    return comm_fail(GLQB_E_INVALID, "comm_all_reduce: %lld floats, the communicator holds %d", (long long)count, c->dev.max_floats);
  if (reinterpret_cast<uintptr_t>(buf_f32) & 3) return comm_fail(GLQB_E_INVALID, "comm_all_reduce: unaligned buffer");
  if (c->dev.world == 1) return GLQB_OK;
  int grid = (int)((count + AR_CHUNK - 1) / AR_CHUNK);
  if (grid > COMM_MAX_UNITS) grid = COMM_MAX_UNITS;
  int chunk = (int)((count + grid - 1) / grid);
  chunk = (chunk + 3) / 4 * 4;
  comm_all_reduce_kernel<<<grid, AR_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(c->dev, reinterpret_cast<float*>(buf_f32),
                                                                                          (int)count, chunk);
  COMM_TRY(cudaGetLastError());
  return GLQB_OK;
}

int glqb_comm_status(GlqbComm* c, int32_t* status_out, int32_t reset) {
  if (!c || !status_out) return comm_fail(GLQB_E_INVALID, "comm_status: null argument");
  int v[3] = {0, 0, 0};                            // epoch, done, status
  COMM_TRY(cudaMemcpy(v, c->base, sizeof(v), cudaMemcpyDeviceToHost));
  *status_out = v[2];
  if (reset && v[2]) {                             // the launch whose wait ran out still closed its epoch
    const int zero = 0;
    COMM_TRY(cudaMemcpy(c->base + 2 * sizeof(int), &zero, sizeof(zero), cudaMemcpyHostToDevice));
  }
  if (v[2]) return comm_fail(GLQB_E_DEVICE, "a wait for a peer rank ran out (status %d): results of that launch are invalid", v[2]);
  return GLQB_OK;
}

int glqb_comm_epoch(GlqbComm* c, int32_t* epoch_out) {
  if (!c || !epoch_out) return comm_fail(GLQB_E_INVALID, "comm_epoch: null argument");
  COMM_TRY(cudaMemcpy(epoch_out, c->base, sizeof(int), cudaMemcpyDeviceToHost));
  return GLQB_OK;
}

void glqb_comm_destroy(GlqbComm* c) {
  if (!c) return;
  for (int r = 0; r < c->dev.world; ++r)
    if (c->peer_ipc[r] && c->peer_base[r]) cudaIpcCloseMemHandle(c->peer_base[r]);
  if (c->base) cudaFree(c->base);
  delete c;
}

}  // extern "C"
