// Device-side building blocks of the NVLink collectives: the per-call context (peer signal pads, epoch, channel),
// system-scope flag stores / polls with a time limit, and the grid-wide exit barrier.
#pragma once

#include "common.cuh"

namespace fsb {

constexpr int kMaxRanks = 8;
// Default limit of one wait for a peer.  Ranks drift apart by far more than a kernel's run time in ordinary training
// (one rank writes a checkpoint, a data loader stalls), so the default is generous; fsb_comm_set_timeout_ms() changes it
// for the process and every kernel launch carries the value that was current when it was launched.
constexpr unsigned long long kCommWaitDefaultNs = 30ull * 1000ull * 1000ull * 1000ull;
// Collective kernels run beside the persistent tensor-core kernels of the compute stream (168 registers x 320 threads
// and ~225 KB of shared memory per SM), so a communication CTA has to fit into what those leave free: 128 threads,
// at most 40 registers per thread and no dynamic shared memory.  A larger CTA cannot become resident until a GEMM CTA
// retires and then keeps the next GEMM off the SM, which serialises communication with compute.
constexpr int COMM_THREADS = 128;
constexpr int COMM_MIN_CTAS_PER_SM = 12;  // caps the kernels at 40 registers per thread
constexpr int COMM_UNROLL = 4;            // independent 16-byte peer loads in flight per thread

struct CommCtx {
  int rank, world;
  uint32_t epoch;             // strictly increasing per call on a channel pair
  int channel;                // base channel; the kernel uses channel (entry) and channel + 1 (exit / mid)
  uint32_t* pads[kMaxRanks];  // peer signal pads: pads[p][channel * kMaxRanks + src]
  unsigned int* counter;      // local scratch counter (zero before the call, left at zero)
  int* status;
  unsigned long long wait_ns; // limit of one wait for a peer
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer16(const void* p) {  // L1-bypassing 16-byte load
  return __ldcg(reinterpret_cast<const uint4*>(p));
}

// Tell every peer that this rank reached `epoch` on `channel` (one thread per peer).
__device__ __forceinline__ void signal_peers(const CommCtx& c, int channel) {
  if (threadIdx.x < c.world) {
    __threadfence_system();
    st_release_sys(c.pads[threadIdx.x] + channel * kMaxRanks + c.rank, c.epoch);
  }
}
// Wait until every peer reached `epoch` on `channel`. Returns false on timeout (status word set).
__device__ __forceinline__ bool wait_peers(const CommCtx& c, int channel) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();
  if (threadIdx.x < c.world) {
    const uint32_t* mine = c.pads[c.rank] + channel * kMaxRanks + threadIdx.x;
    const uint64_t t0 = globaltimer_ns();
    // epochs wrap: compare as signed distance
    while (static_cast<int32_t>(ld_acquire_sys(mine) - c.epoch) < 0) {
      if (globaltimer_ns() - t0 > c.wait_ns) {
        ok_flag = 0;
        if (c.status != nullptr) atomicExch(c.status, FSB_ERR_WAIT_TIMEOUT);
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return ok_flag != 0;
}
// Grid-wide completion: the last CTA to arrive signals the peers on `channel` and waits for theirs.
__device__ __forceinline__ void exit_barrier(const CommCtx& c, int channel) {
  __shared__ int last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(c.counter, 1u);
    last = (prev == gridDim.x - 1) ? 1 : 0;
    if (last) *c.counter = 0;
  }
  __syncthreads();
  if (last) {
    signal_peers(c, channel);
    wait_peers(c, channel);
  }
}

// One pointer per rank (the same window of every rank's symmetric heap).
struct PtrTable { const void* p[kMaxRanks]; };

// exit_barrier for kernels in which only the first `n_ctas` CTAs take part in the collective.
__device__ __forceinline__ void exit_barrier_n(const CommCtx& c, int channel, unsigned int n_ctas) {
  __shared__ int last_n;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(c.counter, 1u);
    last_n = (prev == n_ctas - 1) ? 1 : 0;
    if (last_n) *c.counter = 0;
  }
  __syncthreads();
  if (last_n) {
    signal_peers(c, channel);
    wait_peers(c, channel);
  }
}

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

}  // namespace fsb

// Host side: the process-wide wait limit (one instance per shared object).
namespace fsb_host {
inline unsigned long long& comm_wait_ns() {
  static unsigned long long ns = fsb::kCommWaitDefaultNs;
  return ns;
}
}  // namespace fsb_host
