// Collective kernels over peer-mapped ("symmetric") memory: every rank's arena is
// mapped into every other rank's address space, so a kernel reads and writes its
// peers' HBM directly over NVLink 5 / NVSwitch with ordinary 16-byte loads and
// stores -- no copy engine, no staging through a library.  Cross-rank ordering uses
// per-CTA signal words (st.release.sys / ld.acquire.sys) with monotonically
// increasing epochs, so nothing is ever reset, and every wait is bounded: after the
// limit the kernel records a status word and returns.
//
//   all-reduce   two-shot: copy-in, each rank reduces its 1/W slice from all peers in fp32,
//                applies the scale (1/W for averaging) and the output cast, pushes the slice
//                to every peer, copy-out.  One launch; NVLink traffic 2N(W-1)/W per rank.
//   all-gather   copy-in, then every rank pulls its peers' shards straight into the output.
//   reduce-scatter  copy-in, then rank r pulls slice r from every peer, reduces in fp32 and
//                writes the (optionally cast / scaled) result; a variant applies the sharded
//                AdamW update to the owner's parameter shard in the same pass.
//   all-to-all(v)   pull per-peer slices; MoE dispatch/combine variants fuse the token
//                permutation and the gate-weighted accumulation.
//
// The arena is double-buffered by call parity, so pull-style collectives need no trailing
// barrier: a peer can only overwrite a half two calls later, after this rank has signalled
// that it entered the next call.
// Parity: the reference has no collective kernels (every collective is one vendor-library
// call: reference torch_musa/csrc/distributed/ProcessGroupMCCL.cpp:3250-4291).
#include "comm_common.cuh"

namespace b200k {
using namespace commdev;
namespace {

template <typename T>
__device__ __forceinline__ void copy_packets(T* __restrict__ dst, const T* __restrict__ src, int64_t npk) {
  constexpr int V = Vec16<T>::N;
  constexpr int U = 2 * kUnroll;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; v + (U - 1) * stride < npk; v += U * stride) {
    Vec16<T> r[U];
#pragma unroll
    for (int u = 0; u < U; ++u) r[u] = ld16(src + (v + u * stride) * V);
#pragma unroll
    for (int u = 0; u < U; ++u) st16(dst + (v + u * stride) * V, r[u]);
  }
  for (; v < npk; v += stride) st16(dst + v * V, ld16(src + v * V));
}

// ------------------------------------------------------------------ all-reduce (two-shot)
// arena layout for this call: [in region: n elements of TI][out region: n elements of TO]
template <typename TI, typename TO>
__global__ void __launch_bounds__(kThreads) allreduce_kernel(Peers P, const TI* __restrict__ in, TO* __restrict__ out,
                                                             int64_t n, float scale, uint32_t epoch, int64_t in_off,
                                                             int64_t out_off) {
  constexpr int V = 8;  // packet: 8 elements (16 B of a 16-bit type, 32 B of fp32)
  __shared__ int sh_ok;
  const int W = P.world, r = P.rank;
  const int64_t npk = n / V;                       // host guarantees n % V == 0
  const int64_t chunk = (npk + W - 1) / W;         // packets per rank slice
  const int64_t gstride = (int64_t)gridDim.x * blockDim.x;
  const int64_t g0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  TI* my_in = reinterpret_cast<TI*>(static_cast<char*>(P.buf[r]) + in_off);
  // 1. copy-in, with the same CTA->packet map on every rank
  for (int c = 0; c < W; ++c) {
    const int64_t base = c * chunk, lim = min(chunk, npk - base);
    for (int64_t v = g0; v < lim; v += gstride) {
      const int64_t e = (base + v) * V;
#pragma unroll
      for (int q = 0; q < V * (int)sizeof(TI) / 16; ++q)
        *reinterpret_cast<uint4*>(my_in + e + q * (16 / sizeof(TI))) =
            *reinterpret_cast<const uint4*>(in + e + q * (16 / sizeof(TI)));
    }
  }
  if (!cta_exchange(P, epoch, &sh_ok)) return;
  // 2. reduce my slice from every peer, push the result to every peer's out region
  {
    const int64_t base = r * chunk, lim = min(chunk, npk - base);
    for (int64_t v0 = g0; v0 < lim; v0 += kUnroll * gstride) {
      float acc[kUnroll][V];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
#pragma unroll
        for (int k = 0; k < V; ++k) acc[u][k] = 0.f;
      for (int p = 0; p < W; ++p) {
        const int src = (r + p) % W;  // stagger peers so the W ranks do not hit one GPU at once
        const TI* pin = reinterpret_cast<const TI*>(static_cast<const char*>(P.buf[src]) + in_off);
        TI tmp[kUnroll][V];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int64_t v = v0 + u * gstride;
          if (v < lim) load_packet(pin + (base + v) * V, tmp[u]);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          if (v0 + u * gstride < lim) {
#pragma unroll
            for (int k = 0; k < V; ++k) acc[u][k] += ToF<TI>::to(tmp[u][k]);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t v = v0 + u * gstride;
        if (v < lim) {
#pragma unroll
          for (int k = 0; k < V; ++k) acc[u][k] *= scale;
          for (int p = 0; p < W; ++p) {
            const int dst = (r + p) % W;
            TO* pout = reinterpret_cast<TO*>(static_cast<char*>(P.buf[dst]) + out_off) + (base + v) * V;
            store_acc<TO, V>(pout, acc[u]);
          }
        }
      }
    }
  }
  if (!cta_exchange(P, epoch + 1, &sh_ok)) return;
  // 3. copy-out
  const TO* my_out = reinterpret_cast<const TO*>(static_cast<const char*>(P.buf[r]) + out_off);
  for (int c = 0; c < W; ++c) {
    const int64_t base = c * chunk, lim = min(chunk, npk - base);
    for (int64_t v = g0; v < lim; v += gstride) {
      const int64_t e = (base + v) * V;
#pragma unroll
      for (int q = 0; q < V * (int)sizeof(TO) / 16; ++q)
        *reinterpret_cast<uint4*>(out + e + q * (16 / sizeof(TO))) =
            *reinterpret_cast<const uint4*>(my_out + e + q * (16 / sizeof(TO)));
    }
  }
}

// ------------------------------------------------------------------ all-gather (pull)
// out [W * n] ; arena in region: n elements
template <typename T>
__global__ void __launch_bounds__(kThreads) allgather_kernel(Peers P, const T* __restrict__ in, T* __restrict__ out,
                                                             int64_t n, uint32_t epoch, int64_t in_off) {
  constexpr int V = Vec16<T>::N;
  __shared__ int sh_ok;
  const int W = P.world, r = P.rank;
  const int64_t npk = n / V;
  T* my_in = reinterpret_cast<T*>(static_cast<char*>(P.buf[r]) + in_off);
  copy_packets(my_in, in, npk);
  copy_packets(out + (int64_t)r * n, in, npk);  // own shard: local copy
  if (!cta_exchange(P, epoch, &sh_ok)) return;
  for (int p = 1; p < W; ++p) {
    const int src = (r + p) % W;
    const T* pin = reinterpret_cast<const T*>(static_cast<const char*>(P.buf[src]) + in_off);
    copy_packets(out + (int64_t)src * n, pin, npk);
  }
}

// ------------------------------------------------------------------ reduce-scatter (pull)
// in [W * n] ; out [n] = scale * sum_p in_p[r*n : (r+1)*n]
template <typename TI, typename TO>
__global__ void __launch_bounds__(kThreads) reduce_scatter_kernel(Peers P, const TI* __restrict__ in,
                                                                  TO* __restrict__ out, int64_t n, float scale,
                                                                  uint32_t epoch, int64_t in_off) {
  constexpr int V = 8;
  __shared__ int sh_ok;
  const int W = P.world, r = P.rank;
  const int64_t npk = n / V;
  const int64_t gstride = (int64_t)gridDim.x * blockDim.x;
  const int64_t g0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  TI* my_in = reinterpret_cast<TI*>(static_cast<char*>(P.buf[r]) + in_off);
  // copy-in every slice except my own (nobody else reads it)
  for (int c = 0; c < W; ++c) {
    if (c == r) continue;
    for (int64_t v = g0; v < npk; v += gstride) {
      const int64_t e = ((int64_t)c * npk + v) * V;
#pragma unroll
      for (int q = 0; q < V * (int)sizeof(TI) / 16; ++q)
        *reinterpret_cast<uint4*>(my_in + e + q * (16 / sizeof(TI))) =
            *reinterpret_cast<const uint4*>(in + e + q * (16 / sizeof(TI)));
    }
  }
  if (!cta_exchange(P, epoch, &sh_ok)) return;
  for (int64_t v0 = g0; v0 < npk; v0 += kUnroll * gstride) {
    float acc[kUnroll][V];
    {
      TI tmp[kUnroll][V];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t v = v0 + u * gstride;
        if (v < npk) load_packet(in + ((int64_t)r * npk + v) * V, tmp[u]);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
#pragma unroll
        for (int k = 0; k < V; ++k) acc[u][k] = (v0 + u * gstride < npk) ? ToF<TI>::to(tmp[u][k]) : 0.f;
    }
    for (int p = 1; p < W; ++p) {
      const int src = (r + p) % W;
      const TI* pin = reinterpret_cast<const TI*>(static_cast<const char*>(P.buf[src]) + in_off);
      TI tmp[kUnroll][V];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        const int64_t v = v0 + u * gstride;
        if (v < npk) load_packet(pin + ((int64_t)r * npk + v) * V, tmp[u]);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        if (v0 + u * gstride < npk) {
#pragma unroll
          for (int k = 0; k < V; ++k) acc[u][k] += ToF<TI>::to(tmp[u][k]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int64_t v = v0 + u * gstride;
      if (v < npk) {
#pragma unroll
        for (int k = 0; k < V; ++k) acc[u][k] *= scale;
        store_acc<TO, V>(out + v * V, acc[u]);
      }
    }
  }
}

// reduce-scatter fused with the sharded AdamW step: the reduced gradient never touches memory.
// p32 / m / v : fp32 master shard and moments [n]; p16 (optional): bf16 copy of the updated shard.
template <typename TI>
__global__ void __launch_bounds__(kThreads) reduce_scatter_adamw_kernel(
    Peers P, const TI* __restrict__ in, float* __restrict__ p32, float* __restrict__ m, float* __restrict__ vv,
    __nv_bfloat16* __restrict__ p16, int64_t n, float scale, uint32_t epoch, int64_t in_off, float lr, float beta1,
    float beta2, float eps, float wd, const float* __restrict__ step_ptr) {
  constexpr int V = 8;
  __shared__ int sh_ok;
  const int W = P.world, r = P.rank;
  const int64_t npk = n / V;
  const int64_t gstride = (int64_t)gridDim.x * blockDim.x;
  const int64_t g0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  TI* my_in = reinterpret_cast<TI*>(static_cast<char*>(P.buf[r]) + in_off);
  for (int c = 0; c < W; ++c) {
    if (c == r) continue;
    for (int64_t v = g0; v < npk; v += gstride) {
      const int64_t e = ((int64_t)c * npk + v) * V;
#pragma unroll
      for (int q = 0; q < V * (int)sizeof(TI) / 16; ++q)
        *reinterpret_cast<uint4*>(my_in + e + q * (16 / sizeof(TI))) =
            *reinterpret_cast<const uint4*>(in + e + q * (16 / sizeof(TI)));
    }
  }
  if (!cta_exchange(P, epoch, &sh_ok)) return;
  const float step = *step_ptr;
  const float bc1 = 1.f - powf(beta1, step), bc2s = sqrtf(1.f - powf(beta2, step));
  const float step_size = lr / bc1;
  for (int64_t v = g0; v < npk; v += gstride) {
    const int64_t e = ((int64_t)r * npk + v) * V;
    float g[V];
#pragma unroll
    for (int k = 0; k < V; ++k) g[k] = 0.f;
    for (int p = 0; p < W; ++p) {
      const int src = (r + p) % W;
      const TI* pin = (p == 0) ? in + e : reinterpret_cast<const TI*>(static_cast<const char*>(P.buf[src]) + in_off) + e;
      TI tmp[V];
#pragma unroll
      for (int q = 0; q < V * (int)sizeof(TI) / 16; ++q)
        *reinterpret_cast<uint4*>(tmp + q * (16 / sizeof(TI))) = *reinterpret_cast<const uint4*>(pin + q * (16 / sizeof(TI)));
#pragma unroll
      for (int k = 0; k < V; ++k) g[k] += ToF<TI>::to(tmp[k]);
    }
    const int64_t o = v * V;
    float pf[V], mf[V], vf[V];
#pragma unroll
    for (int k = 0; k < V; k += 4) {
      float4 a = *reinterpret_cast<const float4*>(p32 + o + k), b = *reinterpret_cast<const float4*>(m + o + k),
             c = *reinterpret_cast<const float4*>(vv + o + k);
      pf[k] = a.x; pf[k + 1] = a.y; pf[k + 2] = a.z; pf[k + 3] = a.w;
      mf[k] = b.x; mf[k + 1] = b.y; mf[k + 2] = b.z; mf[k + 3] = b.w;
      vf[k] = c.x; vf[k + 1] = c.y; vf[k + 2] = c.z; vf[k + 3] = c.w;
    }
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const float gr = g[k] * scale;
      pf[k] -= lr * wd * pf[k];
      mf[k] = beta1 * mf[k] + (1.f - beta1) * gr;
      vf[k] = beta2 * vf[k] + (1.f - beta2) * gr * gr;
      pf[k] -= step_size * mf[k] / (sqrtf(vf[k]) / bc2s + eps);
    }
    store_acc<float, V>(p32 + o, pf);
    store_acc<float, V>(m + o, mf);
    store_acc<float, V>(vv + o, vf);
    if (p16) store_acc<__nv_bfloat16, V>(p16 + o, pf);
  }
}

// ------------------------------------------------------------------ all-to-all(v), pull
// in_splits / out_splits / in_offsets / out_offsets in elements, all multiples of the 16-byte packet.
struct A2ASplits {
  int64_t send_off[kMaxWorld];  // where the slice for peer p starts in MY input
  int64_t send_len[kMaxWorld];  // elements sent to peer p
  int64_t recv_off[kMaxWorld];  // where the slice from peer p lands in MY output
  int64_t recv_len[kMaxWorld];  // elements received from peer p
  int64_t peer_send_off[kMaxWorld];  // where MY slice starts in peer p's input (computed by the host from all splits)
};
template <typename T>
__global__ void __launch_bounds__(kThreads) alltoall_kernel(Peers P, const T* __restrict__ in, T* __restrict__ out,
                                                            int64_t n_in, A2ASplits S, uint32_t epoch, int64_t in_off) {
  constexpr int V = Vec16<T>::N;
  __shared__ int sh_ok;
  const int W = P.world, r = P.rank;
  T* my_in = reinterpret_cast<T*>(static_cast<char*>(P.buf[r]) + in_off);
  // Copy in slice by slice with slice-relative packet numbers: packet v of a slice is then written by the same
  // CTA (v modulo the grid) that pulls packet v of it on the receiving rank, which is the only pairing that
  // cta_exchange orders.  Every rank launches the same grid (equal splits).
  (void)n_in;
  for (int p = 0; p < W; ++p)
    if (p != r) copy_packets(my_in + S.send_off[p], in + S.send_off[p], S.send_len[p] / V);
  if (!cta_exchange(P, epoch, &sh_ok)) return;
  for (int p = 0; p < W; ++p) {
    const int src = (r + p) % W;
    const T* pin = (src == r) ? in + S.send_off[r]
                              : reinterpret_cast<const T*>(static_cast<const char*>(P.buf[src]) + in_off) + S.peer_send_off[src];
    copy_packets(out + S.recv_off[src], pin, S.recv_len[src] / V);
  }
}

}  // namespace

namespace commdev {
static std::atomic<long long> g_peer_wait_cycles{4000000000ll};
long long peer_wait_cycles() { return g_peer_wait_cycles.load(std::memory_order_relaxed); }
}  // namespace commdev

static int grid_for(int64_t packets) {
  int64_t b = cdiv(packets, kThreads);
  if (b < 1) b = 1;
  if (b > kMaxChannels) b = kMaxChannels;
  return (int)b;
}

static inline bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace b200k

using namespace b200k;

extern "C" {

int b200_comm_max_world(void) { return kMaxWorld; }
/* SM clock ticks run at up to ~2 GHz: the conversion assumes that rate, so the limit is never shorter than asked */
void b200_comm_set_wait_ms(double ms) {
  long long c = (long long)(ms * 2.0e6);
  if (c < 1000) c = 1000;
  commdev::g_peer_wait_cycles.store(c, std::memory_order_relaxed);
}
double b200_comm_get_wait_ms(void) { return (double)commdev::peer_wait_cycles() / 2.0e6; }
size_t b200_comm_signal_bytes(void) { return (size_t)kPadWords * sizeof(uint32_t); }
int b200_comm_user_word0(void) { return kUserWords; }
int b200_comm_pad_words(void) { return kPadWords; }

#define COMM_DISPATCH2(IN, OUT, TI, TO, ...)                                                       \
  if (IN == B200_F32 && OUT == B200_F32) { using TI = float; using TO = float; __VA_ARGS__; }      \
  else if (IN == B200_BF16 && OUT == B200_BF16) { using TI = __nv_bfloat16; using TO = __nv_bfloat16; __VA_ARGS__; } \
  else if (IN == B200_BF16 && OUT == B200_F32) { using TI = __nv_bfloat16; using TO = float; __VA_ARGS__; }          \
  else if (IN == B200_F32 && OUT == B200_BF16) { using TI = float; using TO = __nv_bfloat16; __VA_ARGS__; }          \
  else if (IN == B200_F16 && OUT == B200_F16) { using TI = __half; using TO = __half; __VA_ARGS__; }                  \
  else if (IN == B200_F16 && OUT == B200_F32) { using TI = __half; using TO = float; __VA_ARGS__; }                   \
  else return (int)cudaErrorNotSupported;

int b200_comm_allreduce(const b200_symm_t* s, int in_dtype, int out_dtype, const void* in, void* out, int64_t n,
                        float scale, uint32_t epoch, int64_t in_off, int64_t out_off, cudaStream_t stream) {
  if (n == 0) return 0;
  if (n % 8 != 0 || !al16(in) || !al16(out) || s->world > kMaxWorld || (in_off & 15) || (out_off & 15))
    return (int)cudaErrorNotSupported;
  Peers P = make_peers(s);
  const int grid = grid_for(n / 8 / s->world + 1);
  COMM_DISPATCH2(in_dtype, out_dtype, TI, TO,
                 (allreduce_kernel<TI, TO><<<grid, kThreads, 0, stream>>>(P, (const TI*)in, (TO*)out, n, scale, epoch,
                                                                          in_off, out_off)));
  B200K_LAUNCH_RET();
}

int b200_comm_allgather(const b200_symm_t* s, int dtype_bytes, const void* in, void* out, int64_t nbytes,
                        uint32_t epoch, int64_t in_off, cudaStream_t stream) {
  (void)dtype_bytes;
  if (nbytes == 0) return 0;
  if (nbytes % 16 != 0 || !al16(in) || !al16(out) || s->world > kMaxWorld || (in_off & 15)) return (int)cudaErrorNotSupported;
  Peers P = make_peers(s);
  // bytes are moved as fp32 packets: the element type does not matter for a gather
  const int64_t n = nbytes / 4;
  allgather_kernel<float><<<grid_for(n / 4), kThreads, 0, stream>>>(P, (const float*)in, (float*)out, n, epoch, in_off);
  B200K_LAUNCH_RET();
}

int b200_comm_reduce_scatter(const b200_symm_t* s, int in_dtype, int out_dtype, const void* in, void* out,
                             int64_t n_out, float scale, uint32_t epoch, int64_t in_off, cudaStream_t stream) {
  if (n_out == 0) return 0;
  if (n_out % 8 != 0 || !al16(in) || !al16(out) || s->world > kMaxWorld || (in_off & 15)) return (int)cudaErrorNotSupported;
  Peers P = make_peers(s);
  const int grid = grid_for(n_out / 8);
  COMM_DISPATCH2(in_dtype, out_dtype, TI, TO,
                 (reduce_scatter_kernel<TI, TO><<<grid, kThreads, 0, stream>>>(P, (const TI*)in, (TO*)out, n_out, scale,
                                                                               epoch, in_off)));
  B200K_LAUNCH_RET();
}

int b200_comm_reduce_scatter_adamw(const b200_symm_t* s, int in_dtype, const void* in, float* p32, float* m, float* v,
                                   void* p16, int64_t n_out, float scale, uint32_t epoch, int64_t in_off, float lr,
                                   float beta1, float beta2, float eps, float wd, const float* step_ptr,
                                   cudaStream_t stream) {
  if (n_out == 0) return 0;
  if (n_out % 8 != 0 || !al16(in) || !al16(p32) || !al16(m) || !al16(v) || (p16 && !al16(p16)) || s->world > kMaxWorld ||
      (in_off & 15))
    return (int)cudaErrorNotSupported;
  Peers P = make_peers(s);
  const int grid = grid_for(n_out / 8);
  if (in_dtype == B200_F32)
    reduce_scatter_adamw_kernel<float><<<grid, kThreads, 0, stream>>>(P, (const float*)in, p32, m, v, (__nv_bfloat16*)p16, n_out, scale, epoch, in_off, lr, beta1, beta2, eps, wd, step_ptr);
  else if (in_dtype == B200_BF16)
    reduce_scatter_adamw_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(P, (const __nv_bfloat16*)in, p32, m, v, (__nv_bfloat16*)p16, n_out, scale, epoch, in_off, lr, beta1, beta2, eps, wd, step_ptr);
  else
    return (int)cudaErrorNotSupported;
  B200K_LAUNCH_RET();
}

int b200_comm_alltoall(const b200_symm_t* s, const void* in, void* out, int64_t in_bytes, const int64_t* send_off,
                       const int64_t* recv_off, const int64_t* recv_len, const int64_t* peer_send_off, uint32_t epoch,
                       int64_t in_off, cudaStream_t stream) {
  if (s->world > kMaxWorld || in_bytes % 16 != 0 || !al16(in) || !al16(out) || (in_off & 15)) return (int)cudaErrorNotSupported;
  A2ASplits S;
  int64_t maxlen = 0;
  for (int i = 0; i < s->world; ++i) {
    if (send_off[i] % 16 || recv_off[i] % 16 || recv_len[i] % 16 || peer_send_off[i] % 16) return (int)cudaErrorNotSupported;
    // byte offsets -> fp32 elements
    S.send_off[i] = send_off[i] / 4; S.recv_off[i] = recv_off[i] / 4; S.recv_len[i] = recv_len[i] / 4;
    S.peer_send_off[i] = peer_send_off[i] / 4;
    const int64_t send_end = i + 1 < s->world ? send_off[i + 1] : in_bytes;
    if (send_end < send_off[i] || (send_end - send_off[i]) % 16) return (int)cudaErrorNotSupported;
    S.send_len[i] = (send_end - send_off[i]) / 4;
    maxlen = std::max(maxlen, recv_len[i]);
  }
  Peers P = make_peers(s);
  // the grid depends on the largest slice only, which equal splits make the same on every rank
  alltoall_kernel<float><<<grid_for(maxlen / 16), kThreads, 0, stream>>>(
      P, (const float*)in, (float*)out, in_bytes / 4, S, epoch, in_off);
  B200K_LAUNCH_RET();
}

}  // extern "C"
