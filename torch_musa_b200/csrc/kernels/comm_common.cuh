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
// Signal pad of one rank, in 32-bit words: [0, kUserWords) per-CTA channel slots of the collectives
// ([channel][source rank]); [kUserWords, kPadWords) words whose layout the owner of the arena chooses
// (kernel-wide flags and counters of the sharded-parameter kernels).
constexpr int kUserWords = kMaxChannels * kMaxWorld;
constexpr int kPadWords = 4 * kUserWords;
// Limit of every cross-rank device wait, in SM clock ticks.  Set by the host (process-group timeout or
// b200_comm_set_wait_ms); a kernel whose wait runs out records a status word and returns.
long long peer_wait_cycles();

struct Peers {
  void* buf[kMaxWorld];
  uint32_t* sig[kMaxWorld];
  int rank, world;
  int* status;  // host-mapped word; set to non-zero when a bounded wait expired
  long long wait_cycles;
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
      if ((++spins & 0xff) == 0 && clock64() - t0 > P.wait_cycles) {
        *sh_ok = 0;
        if (P.status) atomicExch(P.status, 1 + (int)threadIdx.x);
        break;
      }
    }
  }
  __syncthreads();
  return *sh_ok != 0;
}

// 8-element packet load (16 bytes of a 16-bit type, 32 bytes of fp32)
template <typename TI>
__device__ __forceinline__ void load_packet(const TI* __restrict__ p, TI (&tmp)[8]) {
#pragma unroll
  for (int q = 0; q < 8 * (int)sizeof(TI) / 16; ++q)
    *reinterpret_cast<uint4*>(tmp + q * (16 / sizeof(TI))) = *reinterpret_cast<const uint4*>(p + q * (16 / sizeof(TI)));
}

template <typename TO, int V>
__device__ __forceinline__ void store_acc(TO* dst, const float (&acc)[V]) {
  if constexpr (sizeof(TO) == 4) {
#pragma unroll
    for (int k = 0; k < V; k += 4)
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + k) = make_float4(acc[k], acc[k + 1], acc[k + 2], acc[k + 3]);
  } else {
#pragma unroll
    for (int k = 0; k < V; k += 8) {
      Vec16<TO> o;
#pragma unroll
      for (int j = 0; j < 8; ++j) o.v[j] = ToF<TO>::from(acc[k + j]);
      st16(dst + k, o);
    }
  }
}

// Kernel-wide publish: every CTA calls this after its last write of the phase; the CTA that arrives last stores
// `value` into word `word + rank` of every peer's pad (and of its own).  `counter` is a word of the LOCAL pad that
// is zero between launches and that no kernel running at the same time uses.
__device__ __forceinline__ void grid_publish(const Peers& P, uint32_t* counter, int word, uint32_t value) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned prev = atomicAdd(counter, 1u);
    if (prev == gridDim.x - 1) {
      *counter = 0;
      __threadfence_system();
      for (int p = 0; p < P.world; ++p) st_release_sys(P.sig[p] + word + P.rank, value);
    }
  }
}

// All threads of the CTA call this.  Waits until word `word + p` of the local pad has reached `value` for every
// rank p selected by `mask`.  Returns false on time-out (status word = 1 + the rank that did not arrive).
__device__ __forceinline__ bool wait_peers(const Peers& P, int word, uint32_t value, uint32_t mask, int* sh_ok) {
  if (threadIdx.x == 0) *sh_ok = 1;
  __syncthreads();
  if (threadIdx.x < P.world && ((mask >> threadIdx.x) & 1u)) {
    const uint32_t* slot = P.sig[P.rank] + word + threadIdx.x;
    const long long t0 = clock64();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(slot) - value) < 0) {
      if ((++spins & 0xff) == 0 && clock64() - t0 > P.wait_cycles) {
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
  P.wait_cycles = peer_wait_cycles();
  return P;
}

}  // namespace commdev
}  // namespace b200k
