// Shared by the peer-memory collective kernels: the table of mapped peer arenas / signal pads, the
// system-scope release/acquire accessors and the per-CTA cross-rank barrier with a bounded wait.
#pragma once

#include "common.cuh"

namespace b200k {
namespace commdev {

constexpr int kMaxWorld = 16;
constexpr int kMaxChannels = 128;      // CTAs per collective kernel
constexpr int kUnroll = 4;             // packets in flight per thread: peer loads have microseconds of latency
constexpr int kThreads = 512;
constexpr long long kWaitCycles = 4000000000ll;  // ~2 s

struct Peers {
  void* buf[kMaxWorld];
  uint32_t* sig[kMaxWorld];
  int rank, world;
  int* status;  // host-mapped word; set to non-zero when a bounded wait expired
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// All threads of the CTA call this. Publishes this CTA's prior writes to every peer and waits until
// every peer's same-numbered CTA has published epoch `e` too. Returns false on time-out.
__device__ __forceinline__ bool cta_exchange(const Peers& P, uint32_t e, int* sh_ok) {
  __threadfence_system();
  __syncthreads();
  const int ch = blockIdx.x;
  if (threadIdx.x < P.world) {
    const int peer = threadIdx.x;
    // slot [channel][source rank] in the peer's pad
    st_release_sys(P.sig[peer] + ch * kMaxWorld + P.rank, e);
  }
  if (threadIdx.x == 0) *sh_ok = 1;
  __syncthreads();
  if (threadIdx.x < P.world) {
    const uint32_t* slot = P.sig[P.rank] + ch * kMaxWorld + threadIdx.x;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(slot) - e) < 0) {
      if ((++spins & 0xff) == 0 && clock64() - t0 > kWaitCycles) {
        *sh_ok = 0;
        if (P.status) atomicExch(P.status, 1 + (int)threadIdx.x);
        break;
      }
    }
  }
  __syncthreads();
  return *sh_ok != 0;
}


inline Peers make_peers(const b200_symm_t* s) {
  Peers P;
  for (int i = 0; i < kMaxWorld; ++i) {
    P.buf[i] = i < s->world ? s->bufs[i] : nullptr;
    P.sig[i] = i < s->world ? s->sigs[i] : nullptr;
  }
  P.rank = s->rank;
  P.world = s->world;
  P.status = s->status;
  return P;
}

}  // namespace commdev
}  // namespace b200k
