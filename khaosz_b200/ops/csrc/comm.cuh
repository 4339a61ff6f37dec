// Cross-rank synchronisation shared by the in-kernel collectives: peer pointer tables and the
// bounded epoch barrier over a symmetric control buffer (rows of 8 uint32 words per CTA slot).
#pragma once
#include "common.cuh"

namespace kb {
namespace comm {

constexpr int MAX_RANKS = 8;
constexpr int THREADS = 512;

struct Peers {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// All threads of the CTA call this.  Returns false after a timeout (error word set).
static __device__ bool cta_peer_barrier(const Peers& ctrl, int rank, int ws, int slot, uint32_t epoch, int* err,
                                 unsigned long long budget_ns) {
  __shared__ int s_ok;
  __syncthreads();
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < ws) {
    const int peer = threadIdx.x;
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(ctrl.p[peer]) + (size_t)slot * MAX_RANKS + rank, epoch);
    const uint32_t* mine = static_cast<const uint32_t*>(ctrl.p[rank]) + (size_t)slot * MAX_RANKS + peer;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t it = 0;
    // epochs only grow; "at least this epoch" tolerates a peer that already moved on
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      // a peer that is far behind (ranks are not in lockstep) is waited for politely: the polls of a long
      // wait would otherwise compete with the kernels that share the SM and the links
      if (it > 64u) __nanosleep(it > 4096u ? 512 : 64);
      if ((++it & 255u) == 0u && globaltimer_ns() - t0 > budget_ns) {
        s_ok = 0;
        if (err) atomicCAS(err, 0, KB_ERR_TIMEOUT_PEER);
        break;
      }
    }
  }
  __syncthreads();
  return s_ok != 0;
}


}  // namespace comm
}  // namespace kb
