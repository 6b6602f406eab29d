// Expert-parallel MoE token exchange over peer-mapped memory, fused with the permutation and the gate scaling.
//
//   count     slot[t,k] = running index of pair (t,k) inside this rank's batch for expert idx[t,k]; counts[e].
//   dispatch  one kernel: every rank pushes its per-expert counts to all peers and waits for theirs (bounded),
//             derives from the full [world x experts] table where its rows start inside every destination
//             expert's buffer (experts in order, source ranks in order inside an expert), then writes each
//             token row STRAIGHT into the destination GPU's receive buffer over NVLink with 16-byte stores --
//             no send buffer, no separate permute kernel, no all-to-all of split sizes.  pos[t,k] remembers
//             the destination row (-1 when the expert's capacity is exhausted and the pair is dropped).
//   gather    out[t] = sum_k w[t,k] * peer_row(pos[t,k]): the combine.  Pulls the expert outputs from the
//             peers' buffers with 16-byte loads and applies the gate weights in fp32 in registers.  With
//             w == NULL it is the backward of dispatch.
//   scatter   peer_row(pos[t,k]) = w[t,k] * x[t]: the backward of combine (and a dispatch whose positions
//             are already known).
//   gather_dot  dw[t,k] = <g[t], peer_row(pos[t,k])>: the gate gradient.
// Every cross-rank wait is bounded and reports through the arena's status word.
// Parity: the reference has no expert parallelism; its all_to_all is a loop of send/recv pairs
// (reference torch_musa/csrc/distributed/ProcessGroupMCCL.cpp:4022-4117,4119-4224).
#include "comm_common.cuh"

namespace b200k {
using namespace commdev;
namespace {

constexpr int kMoeThreads = 512;
constexpr int kMoeGrid = 96;        // identical on every rank: same-numbered CTAs pair up across ranks
constexpr int kMaxExperts = 256;

__global__ void moe_count_kernel(const int* __restrict__ idx, int* __restrict__ slot, int* __restrict__ counts,
                                 int64_t n_pairs, int E) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_pairs; i += (int64_t)gridDim.x * blockDim.x) {
    const int e = idx[i];
    slot[i] = (e >= 0 && e < E) ? atomicAdd(counts + e, 1) : -1;
  }
}

struct MoeGeom {
  int T, K, d, E, E_local;
  int64_t cap_rows;     // rows of one rank's receive buffer
};

// Row copy by one warp: nvec 16-byte vectors, optional fp32 scale (bf16 payload).
__device__ __forceinline__ void warp_copy_row(__nv_bfloat16* __restrict__ dst, const __nv_bfloat16* __restrict__ src,
                                              int nvec, float scale, bool scaled, int lane) {
  for (int v0 = lane; v0 < nvec; v0 += 32 * 4) {
    Vec16<__nv_bfloat16> r[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (v0 + u * 32 < nvec) r[u] = ld16(src + (int64_t)(v0 + u * 32) * 8);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (v0 + u * 32 < nvec) {
        if (scaled) {
#pragma unroll
          for (int k = 0; k < 8; ++k) r[u].v[k] = __float2bfloat16(__bfloat162float(r[u].v[k]) * scale);
        }
        st16(dst + (int64_t)(v0 + u * 32) * 8, r[u]);
      }
    }
  }
}

__global__ void __launch_bounds__(kMoeThreads)
moe_dispatch_kernel(Peers P, const __nv_bfloat16* __restrict__ x, const int* __restrict__ idx,
                    const int* __restrict__ slot, const int* __restrict__ counts_local, int* __restrict__ pos,
                    int* __restrict__ recv_counts, MoeGeom g, int64_t recv_off, int64_t counts_off, uint32_t epoch) {
  __shared__ int sh_ok;
  __shared__ int sh_start[kMaxExperts];   // first row of my block inside expert e's buffer on its rank
  const int W = P.world, r = P.rank;
  // 1. publish my counts to every peer (every CTA writes the same values, so its own signal covers them)
  for (int i = threadIdx.x; i < W * g.E; i += blockDim.x) {
    const int peer = i / g.E, e = i - peer * g.E;
    int* table = reinterpret_cast<int*>(static_cast<char*>(P.buf[peer]) + counts_off);
    table[r * g.E + e] = counts_local[e];
  }
  if (!cta_exchange(P, epoch, &sh_ok)) return;
  // 2. from the full table: where do my rows start inside each expert's buffer?
  const volatile int* table = reinterpret_cast<const volatile int*>(static_cast<const char*>(P.buf[r]) + counts_off);
  for (int e = threadIdx.x; e < g.E; e += blockDim.x) {
    const int owner = e / g.E_local;
    int start = 0;
    for (int e2 = owner * g.E_local; e2 < e; ++e2)
      for (int s = 0; s < W; ++s) start += table[s * g.E + e2];   // experts before e on the same rank
    for (int s = 0; s < r; ++s) start += table[s * g.E + e];        // sources before me inside expert e
    sh_start[e] = start;
    if (blockIdx.x == 0 && owner == r) {
      int tot = 0;
      for (int s = 0; s < W; ++s) tot += table[s * g.E + e];
      recv_counts[e - r * g.E_local] = tot;
    }
  }
  __syncthreads();
  // 3. write every (token, choice) row into its destination buffer
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int64_t n_pairs = (int64_t)g.T * g.K;
  const int nvec = g.d / 8;
  for (int64_t i = (int64_t)blockIdx.x * wpb + warp; i < n_pairs; i += (int64_t)gridDim.x * wpb) {
    const int e = idx[i];
    int64_t row = -1;
    if (e >= 0 && e < g.E && slot[i] >= 0) {
      row = (int64_t)sh_start[e] + slot[i];
      if (row >= g.cap_rows) row = -1;   // over capacity: dropped
    }
    if (lane == 0) pos[i] = (int)row;
    if (row >= 0) {
      const int owner = e / g.E_local;
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(P.buf[owner]) + recv_off) + row * g.d;
      warp_copy_row(dst, x + (i / g.K) * g.d, nvec, 1.f, false, lane);
    }
  }
  // 4. nobody leaves before every peer's rows have landed here
  cta_exchange(P, epoch + 1, &sh_ok);
}

// out[t] = sum_k w[t,k] * row(pos[t,k]) pulled from the rank that owns expert idx[t,k]
__global__ void __launch_bounds__(kMoeThreads)
moe_gather_kernel(Peers P, __nv_bfloat16* __restrict__ out, const int* __restrict__ idx, const int* __restrict__ pos,
                  const float* __restrict__ w, MoeGeom g, int64_t src_off, uint32_t epoch) {
  __shared__ int sh_ok;
  if (!cta_exchange(P, epoch, &sh_ok)) return;   // the peers' rows are complete
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int nvec = g.d / 8;
  for (int64_t t = (int64_t)blockIdx.x * wpb + warp; t < g.T; t += (int64_t)gridDim.x * wpb) {
    for (int v0 = lane; v0 < nvec; v0 += 32 * 2) {
      float acc[2][8];
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[u][k] = 0.f;
      for (int k = 0; k < g.K; ++k) {
        const int p = pos[t * g.K + k];
        if (p < 0) continue;   // uniform across the warp
        const int owner = idx[t * g.K + k] / g.E_local;
        const float wk = w ? w[t * g.K + k] : 1.f;
        const __nv_bfloat16* src =
            reinterpret_cast<const __nv_bfloat16*>(static_cast<const char*>(P.buf[owner]) + src_off) + (int64_t)p * g.d;
        Vec16<__nv_bfloat16> rr[2];
#pragma unroll
        for (int u = 0; u < 2; ++u)
          if (v0 + u * 32 < nvec) rr[u] = ld16(src + (int64_t)(v0 + u * 32) * 8);
#pragma unroll
        for (int u = 0; u < 2; ++u)
          if (v0 + u * 32 < nvec) {
#pragma unroll
            for (int q = 0; q < 8; ++q) acc[u][q] = fmaf(wk, __bfloat162float(rr[u].v[q]), acc[u][q]);
          }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u)
        if (v0 + u * 32 < nvec) {
          Vec16<__nv_bfloat16> o;
#pragma unroll
          for (int q = 0; q < 8; ++q) o.v[q] = __float2bfloat16(acc[u][q]);
          st16(out + t * g.d + (int64_t)(v0 + u * 32) * 8, o);
        }
    }
  }
}

// row(pos[t,k]) on the owner of expert idx[t,k] = w[t,k] * x[t]
__global__ void __launch_bounds__(kMoeThreads)
moe_scatter_kernel(Peers P, const __nv_bfloat16* __restrict__ x, const int* __restrict__ idx,
                   const int* __restrict__ pos, const float* __restrict__ w, MoeGeom g, int64_t dst_off,
                   uint32_t epoch) {
  __shared__ int sh_ok;
  if (!cta_exchange(P, epoch, &sh_ok)) return;   // the peers no longer read the rows we are about to overwrite
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int64_t n_pairs = (int64_t)g.T * g.K;
  const int nvec = g.d / 8;
  for (int64_t i = (int64_t)blockIdx.x * wpb + warp; i < n_pairs; i += (int64_t)gridDim.x * wpb) {
    const int p = pos[i];
    if (p < 0) continue;
    const int owner = idx[i] / g.E_local;
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(P.buf[owner]) + dst_off) + (int64_t)p * g.d;
    warp_copy_row(dst, x + (i / g.K) * g.d, nvec, w ? w[i] : 1.f, w != nullptr, lane);
  }
  cta_exchange(P, epoch + 1, &sh_ok);
}

// dw[t,k] = <grad[t], row(pos[t,k])>
__global__ void __launch_bounds__(kMoeThreads)
moe_gather_dot_kernel(Peers P, const __nv_bfloat16* __restrict__ grad, const int* __restrict__ idx,
                      const int* __restrict__ pos, float* __restrict__ dw, MoeGeom g, int64_t src_off) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const int64_t n_pairs = (int64_t)g.T * g.K;
  const int nvec = g.d / 8;
  for (int64_t i = (int64_t)blockIdx.x * wpb + warp; i < n_pairs; i += (int64_t)gridDim.x * wpb) {
    const int p = pos[i];
    float s = 0.f;
    if (p >= 0) {
      const int owner = idx[i] / g.E_local;
      const __nv_bfloat16* src =
          reinterpret_cast<const __nv_bfloat16*>(static_cast<const char*>(P.buf[owner]) + src_off) + (int64_t)p * g.d;
      const __nv_bfloat16* gr = grad + (i / g.K) * g.d;
      for (int v0 = lane; v0 < nvec; v0 += 32 * 4) {
        Vec16<__nv_bfloat16> a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (v0 + u * 32 < nvec) {
            a[u] = ld16(src + (int64_t)(v0 + u * 32) * 8);
            b[u] = ld16(gr + (int64_t)(v0 + u * 32) * 8);
          }
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (v0 + u * 32 < nvec) {
#pragma unroll
            for (int q = 0; q < 8; ++q) s = fmaf(__bfloat162float(a[u].v[q]), __bfloat162float(b[u].v[q]), s);
          }
      }
    }
    s = warp_sum(s);
    if (lane == 0) dw[i] = s;
  }
}

bool moe_geom_ok(const b200_symm_t* s, int T, int K, int d, int E) {
  return s && s->world >= 1 && s->world <= kMaxWorld && T >= 0 && K >= 1 && K <= 8 && d > 0 && d % 8 == 0 && E >= 1 &&
         E <= kMaxExperts && E % s->world == 0;
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" {

int b200_moe_count(const int* idx, int* slot, int* counts, int64_t n_pairs, int E, cudaStream_t stream) {
  cudaError_t e = cudaMemsetAsync(counts, 0, sizeof(int) * E, stream);
  if (e != cudaSuccess) return (int)e;
  if (n_pairs == 0) return 0;
  const int grid = (int)std::min<int64_t>((n_pairs + 255) / 256, 1184);
  moe_count_kernel<<<grid, 256, 0, stream>>>(idx, slot, counts, n_pairs, E);
  B200K_LAUNCH_RET();
}

int b200_moe_dispatch(const b200_symm_t* s, const void* x, const int* idx, const int* slot, const int* counts_local,
                      int* pos, int* recv_counts, int T, int K, int d, int E, int64_t cap_rows, int64_t recv_off,
                      int64_t counts_off, uint32_t epoch, cudaStream_t stream) {
  if (!moe_geom_ok(s, T, K, d, E) || (recv_off & 15) || (counts_off & 15) ||
      (reinterpret_cast<uintptr_t>(x) & 15))
    return (int)cudaErrorNotSupported;
  MoeGeom g{T, K, d, E, E / s->world, cap_rows};
  moe_dispatch_kernel<<<kMoeGrid, kMoeThreads, 0, stream>>>(make_peers(s), (const __nv_bfloat16*)x, idx, slot,
                                                            counts_local, pos, recv_counts, g, recv_off, counts_off,
                                                            epoch);
  B200K_LAUNCH_RET();
}

int b200_moe_gather(const b200_symm_t* s, void* out, const int* idx, const int* pos, const float* w, int T, int K,
                    int d, int E, int64_t src_off, uint32_t epoch, cudaStream_t stream) {
  if (!moe_geom_ok(s, T, K, d, E) || (src_off & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return (int)cudaErrorNotSupported;
  MoeGeom g{T, K, d, E, E / s->world, 0};
  moe_gather_kernel<<<kMoeGrid, kMoeThreads, 0, stream>>>(make_peers(s), (__nv_bfloat16*)out, idx, pos, w, g, src_off,
                                                          epoch);
  B200K_LAUNCH_RET();
}

int b200_moe_scatter(const b200_symm_t* s, const void* x, const int* idx, const int* pos, const float* w, int T, int K,
                     int d, int E, int64_t dst_off, uint32_t epoch, cudaStream_t stream) {
  if (!moe_geom_ok(s, T, K, d, E) || (dst_off & 15) || (reinterpret_cast<uintptr_t>(x) & 15))
    return (int)cudaErrorNotSupported;
  MoeGeom g{T, K, d, E, E / s->world, 0};
  moe_scatter_kernel<<<kMoeGrid, kMoeThreads, 0, stream>>>(make_peers(s), (const __nv_bfloat16*)x, idx, pos, w, g,
                                                           dst_off, epoch);
  B200K_LAUNCH_RET();
}

int b200_moe_gather_dot(const b200_symm_t* s, const void* grad, const int* idx, const int* pos, float* dw, int T, int K,
                        int d, int E, int64_t src_off, cudaStream_t stream) {
  if (!moe_geom_ok(s, T, K, d, E) || (src_off & 15) || (reinterpret_cast<uintptr_t>(grad) & 15))
    return (int)cudaErrorNotSupported;
  if ((int64_t)T * K == 0) return 0;
  MoeGeom g{T, K, d, E, E / s->world, 0};
  moe_gather_dot_kernel<<<kMoeGrid, kMoeThreads, 0, stream>>>(make_peers(s), (const __nv_bfloat16*)grad, idx, pos, dw,
                                                              g, src_off);
  B200K_LAUNCH_RET();
}

}  // extern "C"
