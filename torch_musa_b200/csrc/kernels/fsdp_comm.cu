// Sharded-parameter (FSDP2 / ZeRO-3) collectives over peer-mapped memory.
//
// Every rank keeps the low-precision copy of its parameter shards (the "shadow") resident in its symmetric
// arena, laid out as one flat buffer per parameter group.  The three kernels here replace the five passes of the
// library path (cast, copy-in, all-gather, copy-out; copy-in, reduce-scatter, optimizer):
//
//   pack     multi-tensor cast of the fp32 master shards into the shadow, then one kernel-wide flag to all peers
//   gather   waits for the peers' flags and pulls every peer's shadow straight into the FINAL layout of each
//            unsharded parameter (rows [p * shard, (p + 1) * shard) of tensor i come from rank p): no staging
//            buffer on the receiving side and no copy-out pass
//   reduce   pushes slice c of every gradient tensor into rank c's staging slot over NVLink (gradient dtype on the
//            wire, half the bytes of an fp32 reduce-scatter), raises a kernel-wide flag, waits for the peers'
//            flags and sums the W slots of its own slice in fp32; the epilogue either writes the fp32 gradient
//            shard or applies AdamW to the fp32 master shard, both moments and the shadow, and then publishes the
//            shadow's new version, so the reduced gradient never exists in memory
//
// Cross-rank ordering uses kernel-wide flags (the last CTA of a phase publishes with st.release.sys, readers poll
// their own pad with ld.acquire.sys), so no CTA depends on a particular CTA of another rank being resident; every
// wait is bounded and reports through the arena's status word.  With one rank the kernels degenerate to the local
// cast / optimizer pass and touch no flag.
// Parity: the reference patches FSDP2's collectives to call its library all-gather / reduce-scatter and keeps the
// copy-in / copy-out kernels (reference torch_musa/distributed/_composable/fsdp/patch.py:60-194,
// torch_musa/csrc/aten/ops/musa/TensorShape.mu:121,358); it has no fused path.
#include "comm_common.cuh"

namespace b200k {
using namespace commdev;
namespace {

constexpr int kMaxT = B200_FSDP_MAX_TENSORS;
constexpr int kCopyChunk = 65536;   // bytes per work item of the byte movers (8 x 16 B per thread)
constexpr int kRedChunk = 16384;    // elements per work item of the typed kernels (4 packets of 8 per thread)

struct Chunks {
  int n;
  int start[kMaxT + 1];  // prefix sum of the work items per tensor
};

__device__ __forceinline__ int find_tensor(const Chunks& C, int item) {
  int t = 0;
  while (t + 1 < C.n && item >= C.start[t + 1]) ++t;
  return t;
}

// ------------------------------------------------------------------ pack: master shards -> shadow (+ publish)
struct PackArgs {
  const void* src[kMaxT];
  int64_t numel[kMaxT];   // padded shard elements
  int64_t off[kMaxT];     // element offset in the flat shard
  Chunks chunks;
};

template <typename TI, typename TO>
__global__ void __launch_bounds__(kThreads) fsdp_pack_kernel(Peers P, PackArgs A, TO* __restrict__ shadow,
                                                             uint32_t* counter, int flag_word, uint32_t version) {
  const int total = A.chunks.start[A.chunks.n];
  for (int item = blockIdx.x; item < total; item += gridDim.x) {
    const int t = find_tensor(A.chunks, item);
    const int64_t e0 = (int64_t)(item - A.chunks.start[t]) * kRedChunk;
    const int64_t n = min((int64_t)kRedChunk, A.numel[t] - e0);
    const TI* __restrict__ src = static_cast<const TI*>(A.src[t]) + e0;
    TO* __restrict__ dst = shadow + A.off[t] + e0;
    const bool vec = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
    for (int64_t e = (int64_t)threadIdx.x * 8; e < n; e += (int64_t)kThreads * 8) {
      if (vec && e + 8 <= n) {
        TI tmp[8];
        load_packet(src + e, tmp);
        float f[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = ToF<TI>::to(tmp[k]);
        store_acc<TO, 8>(dst + e, f);
      } else {
        for (int k = 0; k < 8 && e + k < n; ++k) dst[e + k] = ToF<TO>::from(ToF<TI>::to(src[e + k]));
      }
    }
  }
  if (P.world > 1) grid_publish(P, counter, flag_word, version);
}

// ------------------------------------------------------------------ gather: peers' shadows -> unsharded tensors
struct GatherArgs {
  char* out[kMaxT];
  int64_t nbytes[kMaxT];  // padded shard bytes of tensor i
  int64_t off[kMaxT];     // byte offset of tensor i in the flat shard (multiple of 16)
  Chunks chunks;          // items per tensor for ONE source rank
};

__global__ void __launch_bounds__(kThreads) fsdp_gather_kernel(Peers P, GatherArgs A, int64_t shadow_off, int flag_word,
                                                               uint32_t version) {
  __shared__ int sh_ok;
  const int W = P.world, r = P.rank;
  if (W > 1) {
    if (!wait_peers(P, flag_word, version, ~(1u << r), &sh_ok)) return;
  }
  const int per_rank = A.chunks.start[A.chunks.n];
  const int64_t total = (int64_t)per_rank * W;
  for (int64_t item = blockIdx.x; item < total; item += gridDim.x) {
    // consecutive CTAs read from different peers
    const int p = (int)((r + 1 + item % W) % W);
    const int c = (int)(item / W);
    const int t = find_tensor(A.chunks, c);
    const int64_t b0 = (int64_t)(c - A.chunks.start[t]) * kCopyChunk;
    const int64_t n = min((int64_t)kCopyChunk, A.nbytes[t] - b0);
    const char* __restrict__ src = static_cast<const char*>(P.buf[p]) + shadow_off + A.off[t] + b0;
    char* __restrict__ dst = A.out[t] + (int64_t)p * A.nbytes[t] + b0;
    if (((reinterpret_cast<uintptr_t>(dst) | (uintptr_t)n) & 15) == 0) {
      const int npk = (int)(n >> 4);
      constexpr int U = kCopyChunk / 16 / kThreads;
      uint4 reg[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = u * kThreads + (int)threadIdx.x;
        if (i < npk) reg[u] = *reinterpret_cast<const uint4*>(src + (int64_t)i * 16);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = u * kThreads + (int)threadIdx.x;
        if (i < npk) *reinterpret_cast<uint4*>(dst + (int64_t)i * 16) = reg[u];
      }
    } else {
      // odd shard sizes: the destination of rank p's rows is not 16-byte aligned; move 2-byte units
      const int64_t nh = n >> 1;
      for (int64_t i = threadIdx.x; i < nh; i += kThreads)
        reinterpret_cast<uint16_t*>(dst)[i] = reinterpret_cast<const uint16_t*>(src)[i];
      if ((n & 1) && threadIdx.x == 0) dst[n - 1] = src[n - 1];
    }
  }
}

// ------------------------------------------------------------------ reduce: gradients -> fp32 shard / AdamW
struct ReduceArgs {
  const void* grad[kMaxT];
  int64_t numel[kMaxT];   // padded shard elements
  int64_t off[kMaxT];     // element offset in the flat shard (multiple of 8)
  int64_t full[kMaxT];    // elements of the unsharded gradient
  Chunks chunks;
  int64_t total;          // flat shard elements (multiple of 8)
};
struct AdamArgs {
  float* p[kMaxT];
  float* m[kMaxT];
  float* v[kMaxT];
  float lr, beta1, beta2, eps, wd, step;
};

// eight elements starting at base[start], zero beyond `limit`
template <typename T>
__device__ __forceinline__ void load8_guarded(const T* __restrict__ base, int64_t start, int64_t limit, bool vec,
                                              T (&out)[8]) {
  if (vec && start + 8 <= limit) {
    load_packet(base + start, out);
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) out[k] = (start + k < limit) ? base[start + k] : ToF<T>::from(0.f);
  }
}

template <typename T>
__device__ __forceinline__ void store_packet(T* dst, const T (&v)[8]) {
#pragma unroll
  for (int q = 0; q < 8 * (int)sizeof(T) / 16; ++q)
    *reinterpret_cast<uint4*>(dst + q * (16 / sizeof(T))) = *reinterpret_cast<const uint4*>(v + q * (16 / sizeof(T)));
}

// MODE 0: out32 (flat fp32 shard) = scale * sum; MODE 1: AdamW on (p, m, v) and the shadow copy
template <typename TI, typename TS, int MODE>
__global__ void __launch_bounds__(kThreads) fsdp_reduce_kernel(Peers P, ReduceArgs A, AdamArgs O, int64_t stage_off,
                                                               float scale, float* __restrict__ out32,
                                                               TS* __restrict__ shadow, uint32_t* counters,
                                                               int ready_word, int ack_word, uint32_t seq,
                                                               uint32_t ack_need, int shadow_word,
                                                               uint32_t shadow_version) {
  __shared__ int sh_ok;
  const int W = P.world, r = P.rank;
  const int per_rank = A.chunks.start[A.chunks.n];
  if (W > 1) {
    // the staging buffer of this call was last used `ring` calls ago: its owners must have finished reading it
    if ((int32_t)ack_need > 0 && !wait_peers(P, ack_word, ack_need, ~(1u << r), &sh_ok)) return;
    // ---- phase 1: push slice c of every gradient to rank c's slot [r]
    const int64_t items = (int64_t)per_rank * (W - 1);
    for (int64_t item = blockIdx.x; item < items; item += gridDim.x) {
      const int c = (int)((r + 1 + item % (W - 1)) % W);
      const int ch = (int)(item / (W - 1));
      const int t = find_tensor(A.chunks, ch);
      const int64_t e0 = (int64_t)(ch - A.chunks.start[t]) * kRedChunk;
      const int64_t n = min((int64_t)kRedChunk, A.numel[t] - e0);
      const TI* __restrict__ g = static_cast<const TI*>(A.grad[t]);
      const bool vec = ((reinterpret_cast<uintptr_t>(g) & 15) == 0) && (A.numel[t] % 8 == 0);
      const int64_t lim = min(A.full[t], (int64_t)(c + 1) * A.numel[t]);
      TI* __restrict__ dst = reinterpret_cast<TI*>(static_cast<char*>(P.buf[c]) + stage_off) + (int64_t)r * A.total +
                             A.off[t] + e0;
      constexpr int U = kRedChunk / 8 / kThreads;
      TI reg[U][8];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t e = ((int64_t)u * kThreads + threadIdx.x) * 8;
        if (e < n) load8_guarded(g, (int64_t)c * A.numel[t] + e0 + e, lim, vec, reg[u]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int64_t e = ((int64_t)u * kThreads + threadIdx.x) * 8;
        if (e < n) store_packet(dst + e, reg[u]);
      }
    }
    grid_publish(P, counters, ready_word, seq);
    // ---- phase 2 needs every peer's slot
    if (!wait_peers(P, ready_word, seq, ~(1u << r), &sh_ok)) return;
  }
  const TI* __restrict__ stage = reinterpret_cast<const TI*>(static_cast<const char*>(P.buf[r]) + stage_off);
  float bc1 = 1.f, bc2s = 1.f, step_size = 0.f;
  if (MODE == 1) {
    bc1 = 1.f - powf(O.beta1, O.step);
    bc2s = sqrtf(1.f - powf(O.beta2, O.step));
    step_size = O.lr / bc1;
  }
  for (int item = blockIdx.x; item < per_rank; item += gridDim.x) {
    const int t = find_tensor(A.chunks, item);
    const int64_t e0 = (int64_t)(item - A.chunks.start[t]) * kRedChunk;
    const int64_t n = min((int64_t)kRedChunk, A.numel[t] - e0);
    const TI* __restrict__ g = static_cast<const TI*>(A.grad[t]);
    const bool vec = ((reinterpret_cast<uintptr_t>(g) & 15) == 0) && (A.numel[t] % 8 == 0);
    const int64_t lim = min(A.full[t], (int64_t)(r + 1) * A.numel[t]);
    constexpr int U = kRedChunk / 8 / kThreads;
#pragma unroll 1
    for (int u0 = 0; u0 < U; u0 += 2) {
      float acc[2][8];
      TI own[2][8];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int64_t e = ((int64_t)(u0 + u) * kThreads + threadIdx.x) * 8;
        if (e < n) load8_guarded(g, (int64_t)r * A.numel[t] + e0 + e, lim, vec, own[u]);
      }
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[u][k] = ToF<TI>::to(own[u][k]);
      for (int q = 1; q < W; ++q) {
        const int s = (r + q) % W;
        const TI* __restrict__ slot = stage + (int64_t)s * A.total + A.off[t] + e0;
        TI tmp[2][8];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int64_t e = ((int64_t)(u0 + u) * kThreads + threadIdx.x) * 8;
          if (e < n) load_packet(slot + e, tmp[u]);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int64_t e = ((int64_t)(u0 + u) * kThreads + threadIdx.x) * 8;
          if (e < n) {
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[u][k] += ToF<TI>::to(tmp[u][k]);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int64_t e = ((int64_t)(u0 + u) * kThreads + threadIdx.x) * 8;
        if (e >= n) continue;
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[u][k] *= scale;
        if (MODE == 0) {
          store_acc<float, 8>(out32 + A.off[t] + e0 + e, acc[u]);   // the flat buffer is padded to whole packets
        } else {
          float* __restrict__ pp = O.p[t] + e0 + e;
          float* __restrict__ pm = O.m[t] + e0 + e;
          float* __restrict__ pv = O.v[t] + e0 + e;
          const bool whole = e + 8 <= n;
          float pf[8], mf[8], vf[8];
          if (whole) {
#pragma unroll
            for (int k = 0; k < 8; k += 4) {
              const float4 a = *reinterpret_cast<const float4*>(pp + k), b = *reinterpret_cast<const float4*>(pm + k),
                           c = *reinterpret_cast<const float4*>(pv + k);
              pf[k] = a.x; pf[k + 1] = a.y; pf[k + 2] = a.z; pf[k + 3] = a.w;
              mf[k] = b.x; mf[k + 1] = b.y; mf[k + 2] = b.z; mf[k + 3] = b.w;
              vf[k] = c.x; vf[k + 1] = c.y; vf[k + 2] = c.z; vf[k + 3] = c.w;
            }
          } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const bool in = e + k < n;
              pf[k] = in ? pp[k] : 0.f; mf[k] = in ? pm[k] : 0.f; vf[k] = in ? pv[k] : 0.f;
            }
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float gr = acc[u][k];
            pf[k] -= O.lr * O.wd * pf[k];
            mf[k] = O.beta1 * mf[k] + (1.f - O.beta1) * gr;
            vf[k] = O.beta2 * vf[k] + (1.f - O.beta2) * gr * gr;
            pf[k] -= step_size * mf[k] / (sqrtf(vf[k]) / bc2s + O.eps);
          }
          if (whole) {
            store_acc<float, 8>(pp, pf);
            store_acc<float, 8>(pm, mf);
            store_acc<float, 8>(pv, vf);
          } else {
            for (int k = 0; k < 8 && e + k < n; ++k) { pp[k] = pf[k]; pm[k] = mf[k]; pv[k] = vf[k]; }
          }
          if (shadow) store_acc<TS, 8>(shadow + A.off[t] + e0 + e, pf);  // padded to whole packets as well
        }
      }
    }
  }
  if (W > 1) {
    // kernel-wide: my slots may be overwritten (ack) and, after the optimizer epilogue, my shadow is current
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned prev = atomicAdd(counters + 1, 1u);
      if (prev == gridDim.x - 1) {
        counters[1] = 0;
        __threadfence_system();
        for (int p = 0; p < W; ++p) {
          st_release_sys(P.sig[p] + ack_word + r, seq);
          if (MODE == 1 && shadow) st_release_sys(P.sig[p] + shadow_word + r, shadow_version);
        }
      }
    }
  }
}

int chunks_for(Chunks& C, int n, const int64_t* sizes, int64_t chunk) {
  C.n = n;
  int64_t acc = 0;
  for (int i = 0; i < n; ++i) {
    C.start[i] = (int)acc;
    acc += cdiv(sizes[i], chunk);
    if (acc > (int64_t)1 << 30) return -1;
  }
  for (int i = n; i <= kMaxT; ++i) C.start[i] = (int)acc;
  return (int)acc;
}

bool layout_ok(const b200_fsdp_layout_t* L) {
  if (!L || L->n < 1 || L->n > kMaxT || (L->total & 7)) return false;
  for (int i = 0; i < L->n; ++i) {
    if (L->shard_numel[i] < 0 || (L->shard_off[i] & 7) || L->shard_off[i] + L->shard_numel[i] > L->total) return false;
    if (i + 1 < L->n && L->shard_off[i + 1] < ((L->shard_off[i] + L->shard_numel[i] + 7) & ~(int64_t)7)) return false;
  }
  return true;
}

int dtype_bytes(int dt) { return dt == B200_F32 ? 4 : (dt == B200_BF16 || dt == B200_F16) ? 2 : 0; }

uint32_t* counter_ptr(const b200_symm_t* s, int word) { return s->sigs[s->rank] + word; }

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" {

int b200_fsdp_pack(const b200_symm_t* s, const b200_fsdp_layout_t* L, const void* const* srcs, int src_dtype,
                   int64_t shadow_off, int dst_dtype, int flag_word, uint32_t version, int counter_word, int n_ctas,
                   cudaStream_t stream) {
  if (!layout_ok(L) || (shadow_off & 15) || s->world > kMaxWorld || n_ctas < 1) return (int)cudaErrorInvalidValue;
  PackArgs A;
  for (int i = 0; i < L->n; ++i) { A.src[i] = srcs[i]; A.numel[i] = L->shard_numel[i]; A.off[i] = L->shard_off[i]; }
  const int items = chunks_for(A.chunks, L->n, L->shard_numel, kRedChunk);
  if (items < 0) return (int)cudaErrorInvalidValue;
  Peers P = make_peers(s);
  void* shadow = static_cast<char*>(s->bufs[s->rank]) + shadow_off;
  const int grid = std::max(1, std::min(n_ctas, std::max(items, 1)));
  uint32_t* counter = counter_ptr(s, counter_word);
#define PACK(TI, TO) fsdp_pack_kernel<TI, TO><<<grid, kThreads, 0, stream>>>(P, A, (TO*)shadow, counter, flag_word, version)
  if (src_dtype == B200_F32 && dst_dtype == B200_BF16) PACK(float, __nv_bfloat16);
  else if (src_dtype == B200_F32 && dst_dtype == B200_F16) PACK(float, __half);
  else if (src_dtype == B200_F32 && dst_dtype == B200_F32) PACK(float, float);
  else if (src_dtype == B200_BF16 && dst_dtype == B200_BF16) PACK(__nv_bfloat16, __nv_bfloat16);
  else if (src_dtype == B200_F16 && dst_dtype == B200_F16) PACK(__half, __half);
  else return (int)cudaErrorNotSupported;
#undef PACK
  B200K_LAUNCH_RET();
}

int b200_fsdp_gather(const b200_symm_t* s, const b200_fsdp_layout_t* L, void* const* outs, int dtype,
                     int64_t shadow_off, int flag_word, uint32_t version, int n_ctas, cudaStream_t stream) {
  const int eb = dtype_bytes(dtype);
  if (!layout_ok(L) || !eb || (shadow_off & 15) || s->world > kMaxWorld || n_ctas < 1) return (int)cudaErrorInvalidValue;
  GatherArgs A;
  int64_t nb[kMaxT];
  for (int i = 0; i < L->n; ++i) {
    A.out[i] = static_cast<char*>(outs[i]);
    A.nbytes[i] = nb[i] = L->shard_numel[i] * eb;
    A.off[i] = L->shard_off[i] * eb;
  }
  const int items = chunks_for(A.chunks, L->n, nb, kCopyChunk);
  if (items < 0) return (int)cudaErrorInvalidValue;
  if (items == 0) return 0;
  Peers P = make_peers(s);
  const int grid = (int)std::max<int64_t>(1, std::min<int64_t>(n_ctas, (int64_t)items * s->world));
  fsdp_gather_kernel<<<grid, kThreads, 0, stream>>>(P, A, shadow_off, flag_word, version);
  B200K_LAUNCH_RET();
}

int b200_fsdp_reduce(const b200_symm_t* s, const b200_fsdp_layout_t* L, const void* const* grads, int grad_dtype,
                     int64_t stage_off, float scale, float* out32, const b200_fsdp_adamw_t* opt, int ready_word,
                     int ack_word, uint32_t seq, uint32_t ack_need, int counter_word, int n_ctas, cudaStream_t stream) {
  if (!layout_ok(L) || (stage_off & 15) || s->world > kMaxWorld || n_ctas < 1 || (!out32 && !opt) || (out32 && opt))
    return (int)cudaErrorInvalidValue;
  if (out32 && (reinterpret_cast<uintptr_t>(out32) & 15)) return (int)cudaErrorInvalidValue;
  ReduceArgs A;
  AdamArgs O{};
  for (int i = 0; i < L->n; ++i) {
    A.grad[i] = grads[i];
    A.numel[i] = L->shard_numel[i];
    A.off[i] = L->shard_off[i];
    A.full[i] = L->full_numel[i];
    if (opt) {
      O.p[i] = opt->p[i]; O.m[i] = opt->m[i]; O.v[i] = opt->v[i];
      if (((reinterpret_cast<uintptr_t>(O.p[i]) | reinterpret_cast<uintptr_t>(O.m[i]) |
            reinterpret_cast<uintptr_t>(O.v[i])) & 15) != 0)
        return (int)cudaErrorInvalidValue;
    }
  }
  A.total = L->total;
  const int items = chunks_for(A.chunks, L->n, L->shard_numel, kRedChunk);
  if (items < 0) return (int)cudaErrorInvalidValue;
  if (items == 0) return 0;
  void* shadow = nullptr;
  int shadow_dtype = B200_BF16, shadow_word = 0;
  uint32_t shadow_version = 0;
  if (opt) {
    O.lr = opt->lr; O.beta1 = opt->beta1; O.beta2 = opt->beta2; O.eps = opt->eps; O.wd = opt->weight_decay; O.step = opt->step;
    if (opt->shadow_off >= 0) {
      if (opt->shadow_off & 15) return (int)cudaErrorInvalidValue;
      shadow = static_cast<char*>(s->bufs[s->rank]) + opt->shadow_off;
      shadow_dtype = opt->shadow_dtype;
      shadow_word = opt->shadow_flag_word;
      shadow_version = opt->shadow_version;
    }
  }
  Peers P = make_peers(s);
  const int grid = std::max(1, std::min(n_ctas, items * std::max(1, s->world - 1)));
  uint32_t* counters = counter_ptr(s, counter_word);
#define RED(TI, TS, MODE)                                                                                          \
  fsdp_reduce_kernel<TI, TS, MODE><<<grid, kThreads, 0, stream>>>(P, A, O, stage_off, scale, out32, (TS*)shadow,    \
                                                                  counters, ready_word, ack_word, seq, ack_need,     \
                                                                  shadow_word, shadow_version)
  if (!opt) {
    if (grad_dtype == B200_BF16) RED(__nv_bfloat16, __nv_bfloat16, 0);
    else if (grad_dtype == B200_F16) RED(__half, __half, 0);
    else if (grad_dtype == B200_F32) RED(float, float, 0);
    else return (int)cudaErrorNotSupported;
  } else if (shadow_dtype == B200_BF16) {
    if (grad_dtype == B200_BF16) RED(__nv_bfloat16, __nv_bfloat16, 1);
    else if (grad_dtype == B200_F32) RED(float, __nv_bfloat16, 1);
    else return (int)cudaErrorNotSupported;
  } else if (shadow_dtype == B200_F16) {
    if (grad_dtype == B200_F16) RED(__half, __half, 1);
    else if (grad_dtype == B200_F32) RED(float, __half, 1);
    else return (int)cudaErrorNotSupported;
  } else {
    return (int)cudaErrorNotSupported;
  }
#undef RED
  B200K_LAUNCH_RET();
}

}  // extern "C"
