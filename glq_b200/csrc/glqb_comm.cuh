// One-shot sum over tensor-parallel ranks inside a kernel, for messages of a few KB to a few hundred KB.
//
// Every rank owns one receive area, mapped into the address space of all ranks of the node.  A CTA that holds a piece
// of its rank's partial result stores it into the receive area of EVERY rank (plain stores through NVLink, its own
// area included), then raises one flag per peer; it waits until every peer's flag for the same piece has arrived in
// its own memory and adds the pieces up in rank order 0..G-1, so all ranks obtain the same bits.  Nothing is read
// from a peer: a store travels one way, a load would travel both.  There is no bulk-tensor copy and no multicast
// load anywhere in this path.
//
// Flags carry the launch's epoch (launches that use the communicator, counted on the device by the kernels
// themselves, so a replayed CUDA graph needs no changing argument); areas are double-buffered by epoch parity.  Why
// two suffice: a rank overwrites parity p in launch e + 2, which ends only after launch e + 1 has received every
// peer's flag, and a peer raises flags of launch e + 1 only after its own launch e (the last reader of parity p) has
// completed in stream order.
//
// Every wait is bounded by the communicator's time limit; when it runs out the CTA records ST_GAVE_UP_PEER in the
// status word and carries on with what has arrived (the host reads the status; the context stays usable).
#pragma once
#include <stdint.h>

namespace glqb {

constexpr int COMM_MAX_RANKS = 8;
constexpr int COMM_MAX_UNITS = 256;      // pieces (output blocks, chunks) one launch may exchange
constexpr int COMM_CTRL_BYTES = 256;     // epoch, done, status at the head of the area

struct CommDev {
  float* data[COMM_MAX_RANKS];           // rank r's receive area as mapped here: [2 parities][world sources][max_floats]
  int* flags[COMM_MAX_RANKS];            // rank r's flags as mapped here: [2][world][COMM_MAX_UNITS]
  int* epoch;                            // local: launches completed so far
  int* done;                             // local: CTAs of the running launch that have finished
  int* status;                           // local status word
  long long wait_ns;                     // limit of every wait
  int rank, world, max_floats;
};

#ifdef __CUDACC__
__device__ __forceinline__ unsigned long long comm_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// The epoch of the running launch.  Read it only after the previous kernel of the stream has completed (after
// griddepcontrol.wait in a kernel launched with programmatic stream serialization).
__device__ __forceinline__ int comm_epoch(const CommDev& C) {
  return *reinterpret_cast<volatile int*>(C.epoch) + 1;
}

__device__ __forceinline__ float* comm_slot(const CommDev& C, int owner, int e, int src) {
  return C.data[owner] + ((size_t)((e & 1) * C.world + src)) * (size_t)C.max_floats;
}

// After all threads of the CTA have stored their piece into every rank's area: raise the flags, wait for the peers'.
// `unit` names the piece (the same number on every rank).  Ends with a barrier: afterwards every thread may read all
// sources of the piece from the local area.
__device__ __forceinline__ void comm_signal_and_wait(const CommDev& C, int e, int unit) {
  __syncthreads();
  const int t = threadIdx.x;
  if (t < C.world && t != C.rank) {
    __threadfence_system();              // the CTA's stores (ordered before this thread by the barrier) before the flag
    int* remote = C.flags[t] + ((e & 1) * C.world + C.rank) * COMM_MAX_UNITS + unit;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(remote), "r"(e) : "memory");
    const int* mine = C.flags[C.rank] + ((e & 1) * C.world + t) * COMM_MAX_UNITS + unit;
    const unsigned long long t0 = comm_now_ns();
    for (unsigned it = 0;; ++it) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
      if (v >= e) break;
      if ((it & 31u) == 31u && (long long)(comm_now_ns() - t0) > C.wait_ns) {
        atomicCAS(C.status, 0, 6 /* ST_GAVE_UP_PEER */);
        break;
      }
    }
  }
  __syncthreads();
}

// Last statement of every CTA of a launch that uses the communicator: the last one to arrive closes the epoch.
__device__ __forceinline__ void comm_cta_done(const CommDev& C, int e) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const int old = atomicAdd(C.done, 1);
    if (old == (int)(gridDim.x * gridDim.y * gridDim.z) - 1) {
      *reinterpret_cast<volatile int*>(C.done) = 0;
      __threadfence();
      *reinterpret_cast<volatile int*>(C.epoch) = e;
    }
  }
}
#endif

}  // namespace glqb
