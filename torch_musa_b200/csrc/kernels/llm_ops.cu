// Fused transformer helper kernels: rotary embedding, SwiGLU (packed and
// two-tensor forms) forward/backward, embedding gather and its two backward
// strategies (fp32 atomics; deterministic sorted segments), Philox dropout and
// random fills.  All are bandwidth-bound: 128-bit accesses, grid capped at a few
// waves over the 148 SMs.
// Parity: reference torch_musa/csrc/aten/ops/RoPE.cpp:68-160, SwiGlu.cpp:70-115,
// musa/GatedSilu.mu:24-40, musa/Embedding.mu:20, musa/EmbeddingBackwardKernel.mu,
// Dropout.cpp:107-131.
#include "common.cuh"

namespace b200k {
namespace {

constexpr int kThreads = 256;

inline int grid_cap(int64_t work_items) {
  int64_t b = cdiv(work_items, kThreads);
  int64_t cap = (int64_t)kSMs * 8;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

// ------------------------------------------------------------------- RoPE
// one thread handles one 16-byte vector of the first half and its partner in the second half
// (half layout) or one vector of interleaved pairs.
template <typename T, bool INTERLEAVED>
__global__ void __launch_bounds__(kThreads) rope_kernel(T* __restrict__ out, const T* __restrict__ x,
                                                        const float* __restrict__ cosv, const float* __restrict__ sinv,
                                                        const int64_t* __restrict__ pos, int64_t tokens, int64_t seq,
                                                        int heads, int dim, int64_t ts, int64_t hs, float sign) {
  constexpr int V = Vec16<T>::N;
  const int half = dim / 2;
  const int vec_per_head = INTERLEAVED ? dim / V : half / V;
  const int64_t total = tokens * heads * vec_per_head;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int v = (int)(i % vec_per_head);
    int64_t th = i / vec_per_head;
    int h = (int)(th % heads);
    int64_t t = th / heads;
    int64_t p = pos ? pos[t] : (t % seq);
    const T* xp = x + t * ts + (int64_t)h * hs;
    T* op = out + (t * heads + h) * (int64_t)dim;
    const float* cp = cosv + p * half;
    const float* sp = sinv + p * half;
    if constexpr (INTERLEAVED) {
      Vec16<T> a = ld16(xp + v * V), o;
#pragma unroll
      for (int k = 0; k < V; k += 2) {
        int j = (v * V + k) / 2;
        float c = cp[j], s = sp[j] * sign;
        float x0 = ToF<T>::to(a.v[k]), x1 = ToF<T>::to(a.v[k + 1]);
        o.v[k] = ToF<T>::from(x0 * c - x1 * s);
        o.v[k + 1] = ToF<T>::from(x1 * c + x0 * s);
      }
      st16(op + v * V, o);
    } else {
      Vec16<T> a = ld16(xp + v * V), b = ld16(xp + half + v * V), oa, ob;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        int j = v * V + k;
        float c = cp[j], s = sp[j] * sign;
        float x0 = ToF<T>::to(a.v[k]), x1 = ToF<T>::to(b.v[k]);
        oa.v[k] = ToF<T>::from(x0 * c - x1 * s);
        ob.v[k] = ToF<T>::from(x1 * c + x0 * s);
      }
      st16(op + v * V, oa);
      st16(op + half + v * V, ob);
    }
  }
}

// ------------------------------------------------------------------- SwiGLU
__device__ __forceinline__ float silu_f(float g) { return g / (1.f + __expf(-g)); }

// One CTA per (row, chunk of kSwU * blockDim vectors): no index division, four independent gate / up loads in
// flight per thread before the first use.
constexpr int kSwU = 4;
constexpr int kSwThreads = 128;

// Packed row groups whose lengths live on the device (the rows a mixture-of-experts layer received): only the
// first sum(counts) rows carry data.  Every thread adds the few counts itself (they sit in L2).
__device__ __forceinline__ int64_t live_rows(const int* __restrict__ counts, int n) {
  int64_t s = 0;
  for (int i = 0; i < n; ++i) s += max(__ldg(counts + i), 0);
  return s;
}

template <typename T>
__global__ void __launch_bounds__(kSwThreads) swiglu_fwd_kernel(T* __restrict__ out, const T* __restrict__ x,
                                                                int64_t rows, int64_t h,
                                                                const int* __restrict__ row_counts, int n_counts) {
  constexpr int V = Vec16<T>::N;
  const int vh = (int)(h / V);
  const int64_t r = blockIdx.x;
  if (row_counts && r >= live_rows(row_counts, n_counts)) return;   // rows of no group: left untouched
  const T* gp = x + r * 2 * h;
  const T* up = gp + h;
  T* op = out + r * h;
  const int v0 = blockIdx.y * (kSwThreads * kSwU) + threadIdx.x;
  Vec16<T> g[kSwU], u[kSwU];
#pragma unroll
  for (int k = 0; k < kSwU; ++k) {
    const int v = v0 + k * kSwThreads;
    if (v < vh) { g[k] = ld16_stream(gp + (int64_t)v * V); u[k] = ld16_stream(up + (int64_t)v * V); }
  }
#pragma unroll
  for (int k = 0; k < kSwU; ++k) {
    const int v = v0 + k * kSwThreads;
    if (v < vh) {
      Vec16<T> o;
#pragma unroll
      for (int e = 0; e < V; ++e) o.v[e] = ToF<T>::from(silu_f(ToF<T>::to(g[k].v[e])) * ToF<T>::to(u[k].v[e]));
      st16_stream(op + (int64_t)v * V, o);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kSwThreads) swiglu_bwd_kernel(T* __restrict__ dx, const T* __restrict__ dy,
                                                                const T* __restrict__ x, int64_t rows, int64_t h,
                                                                const int* __restrict__ row_counts, int n_counts) {
  constexpr int V = Vec16<T>::N;
  const int vh = (int)(h / V);
  const int64_t r = blockIdx.x;
  if (row_counts && r >= live_rows(row_counts, n_counts)) return;
  const T* gp = x + r * 2 * h;
  const T* up = gp + h;
  const T* dp = dy + r * h;
  T* dgp = dx + r * 2 * h;
  T* dup = dgp + h;
  const int v0 = blockIdx.y * (kSwThreads * kSwU) + threadIdx.x;
  Vec16<T> g[kSwU], u[kSwU], d[kSwU];
#pragma unroll
  for (int k = 0; k < kSwU; ++k) {
    const int v = v0 + k * kSwThreads;
    if (v < vh) {
      g[k] = ld16_stream(gp + (int64_t)v * V);
      u[k] = ld16_stream(up + (int64_t)v * V);
      d[k] = ld16_stream(dp + (int64_t)v * V);
    }
  }
#pragma unroll
  for (int k = 0; k < kSwU; ++k) {
    const int v = v0 + k * kSwThreads;
    if (v < vh) {
      Vec16<T> dg, du;
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float gf = ToF<T>::to(g[k].v[e]), uf = ToF<T>::to(u[k].v[e]), df = ToF<T>::to(d[k].v[e]);
        const float sg = 1.f / (1.f + __expf(-gf));
        dg.v[e] = ToF<T>::from(df * uf * sg * (1.f + gf * (1.f - sg)));
        du.v[e] = ToF<T>::from(df * gf * sg);
      }
      st16_stream(dgp + (int64_t)v * V, dg);
      st16_stream(dup + (int64_t)v * V, du);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) silu_mul_fwd_kernel(T* __restrict__ out, const T* __restrict__ gate,
                                                                const T* __restrict__ up, int64_t n) {
  constexpr int V = Vec16<T>::N;
  const int64_t nvec = n / V;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    Vec16<T> g = ld16_stream(gate + i * V), u = ld16_stream(up + i * V), o;
#pragma unroll
    for (int k = 0; k < V; ++k) o.v[k] = ToF<T>::from(silu_f(ToF<T>::to(g.v[k])) * ToF<T>::to(u.v[k]));
    st16_stream(out + i * V, o);
  }
  int64_t t = nvec * V + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t < n) out[t] = ToF<T>::from(silu_f(ToF<T>::to(gate[t])) * ToF<T>::to(up[t]));
}

template <typename T>
__global__ void __launch_bounds__(kThreads) silu_mul_bwd_kernel(T* __restrict__ dgate, T* __restrict__ dup,
                                                                const T* __restrict__ dy, const T* __restrict__ gate,
                                                                const T* __restrict__ up, int64_t n) {
  constexpr int V = Vec16<T>::N;
  const int64_t nvec = n / V;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) {
    Vec16<T> g = ld16_stream(gate + i * V), u = ld16_stream(up + i * V), d = ld16_stream(dy + i * V), dg, du;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float gf = ToF<T>::to(g.v[k]), uf = ToF<T>::to(u.v[k]), df = ToF<T>::to(d.v[k]);
      float s = 1.f / (1.f + __expf(-gf));
      dg.v[k] = ToF<T>::from(df * uf * s * (1.f + gf * (1.f - s)));
      du.v[k] = ToF<T>::from(df * gf * s);
    }
    st16_stream(dgate + i * V, dg);
    st16_stream(dup + i * V, du);
  }
  int64_t t = nvec * V + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t < n) {
    float gf = ToF<T>::to(gate[t]), uf = ToF<T>::to(up[t]), df = ToF<T>::to(dy[t]);
    float s = 1.f / (1.f + __expf(-gf));
    dgate[t] = ToF<T>::from(df * uf * s * (1.f + gf * (1.f - s)));
    dup[t] = ToF<T>::from(df * gf * s);
  }
}

// ------------------------------------------------------------------- embedding
template <typename T>
__global__ void __launch_bounds__(kThreads) embedding_fwd_kernel(T* __restrict__ out, const T* __restrict__ w,
                                                                 const int64_t* __restrict__ idx, int64_t n,
                                                                 int64_t dim, int64_t vocab) {
  constexpr int V = Vec16<T>::N;
  const int64_t vd = dim / V, total = n * vd;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / vd, c = (i % vd) * V;
    int64_t t = idx[r];
    Vec16<T> v;
    if (t >= 0 && t < vocab) v = ld16(w + t * dim + c);
    else {
#pragma unroll
      for (int k = 0; k < V; ++k) v.v[k] = ToF<T>::from(0.f);
    }
    st16_stream(out + r * dim + c, v);
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) embedding_bwd_atomic_kernel(float* __restrict__ gw,
                                                                        const T* __restrict__ go,
                                                                        const int64_t* __restrict__ idx, int64_t n,
                                                                        int64_t dim, int64_t vocab, int64_t pad) {
  const int64_t total = n * dim;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    int64_t r = i / dim, c = i % dim;
    int64_t t = idx[r];
    if (t == pad || t < 0 || t >= vocab) continue;
    atomicAdd(gw + t * dim + c, ToF<T>::to(go[i]));
  }
}

// One CTA per run of equal sorted indices would need a segment table; instead every CTA handles a
// (row-of-sorted-list, column-strip) pair and only the first row of each run does the summation,
// walking forward over its run.  Deterministic: the order of addition is the sorted order.
template <typename T>
__global__ void __launch_bounds__(128) embedding_bwd_sorted_kernel(T* __restrict__ gw, const T* __restrict__ go,
                                                                   const int64_t* __restrict__ sidx,
                                                                   const int64_t* __restrict__ perm, int64_t n,
                                                                   int64_t dim, int64_t vocab, int64_t pad) {
  const int64_t r = blockIdx.x;
  const int64_t t = sidx[r];
  if (r > 0 && sidx[r - 1] == t) return;  // not a run head
  if (t == pad || t < 0 || t >= vocab) return;
  for (int64_t c = (int64_t)blockIdx.y * blockDim.x + threadIdx.x; c < dim; c += (int64_t)gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int64_t q = r; q < n && sidx[q] == t; ++q) acc += ToF<T>::to(go[perm[q] * dim + c]);
    gw[t * dim + c] = ToF<T>::from(acc);
  }
}

// ------------------------------------------------------------------- Philox 4x32-10
struct Philox {
  uint2 key;
  uint4 ctr;
  __device__ Philox(uint64_t seed, uint64_t subseq, uint64_t offset) {
    key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
    ctr = make_uint4((uint32_t)offset, (uint32_t)(offset >> 32), (uint32_t)subseq, (uint32_t)(subseq >> 32));
  }
  __device__ __forceinline__ uint4 next() {
    uint4 c = ctr;
    uint2 k = key;
#pragma unroll
    for (int i = 0; i < 10; ++i) {
      uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
      uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
      c = make_uint4(hi1 ^ c.y ^ k.x, lo1, hi0 ^ c.w ^ k.y, lo0);
      k.x += 0x9E3779B9u;
      k.y += 0xBB67AE85u;
    }
    // advance the 128-bit counter by one
    if (++ctr.x == 0) if (++ctr.y == 0) if (++ctr.z == 0) ++ctr.w;
    return c;
  }
};
__device__ __forceinline__ float u01(uint32_t x) { return ((float)(x >> 8) + 0.5f) * (1.0f / 16777216.0f); }

__device__ __forceinline__ void unpack(const b200_philox_t& r, uint64_t& seed, uint64_t& offset) {
  if (r.captured) {
    seed = (uint64_t)(*r.seed_ptr);
    offset = (uint64_t)(*r.offset_ptr) + r.offset_intragraph;
  } else {
    seed = r.seed;
    offset = r.offset;
  }
}

// each thread owns elements [4*tid, 4*tid+4) of every (gridsize*4)-element round; one Philox call per round
template <typename T>
__global__ void __launch_bounds__(kThreads) dropout_fwd_kernel(T* __restrict__ out, uint8_t* __restrict__ mask,
                                                               const T* __restrict__ x, int64_t n, float p,
                                                               b200_philox_t rng) {
  uint64_t seed, offset;
  unpack(rng, seed, offset);
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  Philox ph(seed, (uint64_t)tid, offset / 4);
  const float scale = 1.f / (1.f - p);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
  for (int64_t base = tid * 4; base < n; base += stride) {
    uint4 r = ph.next();
    uint32_t rr[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      int64_t i = base + k;
      if (i < n) {
        bool keep = u01(rr[k]) >= p;
        out[i] = ToF<T>::from(keep ? ToF<T>::to(x[i]) * scale : 0.f);
        if (mask) mask[i] = keep ? 1 : 0;
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads) dropout_bwd_kernel(T* __restrict__ dx, const T* __restrict__ dy,
                                                               const uint8_t* __restrict__ mask, int64_t n, float scale) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    dx[i] = ToF<T>::from(mask[i] ? ToF<T>::to(dy[i]) * scale : 0.f);
}

template <typename T, bool NORMAL>
__global__ void __launch_bounds__(kThreads) random_fill_kernel(T* __restrict__ out, int64_t n, float a, float b,
                                                               b200_philox_t rng) {
  uint64_t seed, offset;
  unpack(rng, seed, offset);
  const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  Philox ph(seed, (uint64_t)tid, offset / 4);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x * 4;
  for (int64_t base = tid * 4; base < n; base += stride) {
    uint4 r = ph.next();
    float v[4];
    if constexpr (NORMAL) {
      float u0 = u01(r.x), u1 = u01(r.y), u2 = u01(r.z), u3 = u01(r.w);
      float r0 = sqrtf(-2.f * __logf(u0)), r1 = sqrtf(-2.f * __logf(u2));
      float s0, c0, s1, c1;
      __sincosf(6.283185307179586f * u1, &s0, &c0);
      __sincosf(6.283185307179586f * u3, &s1, &c1);
      v[0] = a + b * r0 * c0; v[1] = a + b * r0 * s0; v[2] = a + b * r1 * c1; v[3] = a + b * r1 * s1;
    } else {
      v[0] = a + (b - a) * u01(r.x); v[1] = a + (b - a) * u01(r.y);
      v[2] = a + (b - a) * u01(r.z); v[3] = a + (b - a) * u01(r.w);
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) if (base + k < n) out[base + k] = ToF<T>::from(v[k]);
  }
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" {

uint64_t b200_philox_increment(int64_t n) {
  // one Philox call (4 outputs) per thread per grid-stride round; worst case is the smallest grid
  int64_t quads = cdiv(n, 4);
  int grid = grid_cap(quads);
  int64_t rounds = cdiv(quads, (int64_t)grid * kThreads);
  return (uint64_t)(rounds < 1 ? 1 : rounds) * 4;
}

int b200_rope(int dtype, void* out, const void* x, const float* cosv, const float* sinv, const int64_t* pos,
              int64_t tokens, int64_t seq, int heads, int dim, int64_t ts, int64_t hs, int interleaved, int conj,
              cudaStream_t stream) {
  if (tokens == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    constexpr int V = Vec16<T>::N;
    if (dim % 2 != 0 || (dim / 2) % V != 0 || ts % V != 0 || hs % V != 0 || !aligned16((const T*)x) || !aligned16((T*)out))
      return (int)cudaErrorNotSupported;
    int64_t work = tokens * heads * (interleaved ? dim / V : dim / 2 / V);
    float sign = conj ? -1.f : 1.f;
    if (interleaved)
      rope_kernel<T, true><<<grid_cap(work), kThreads, 0, stream>>>((T*)out, (const T*)x, cosv, sinv, pos, tokens, seq, heads, dim, ts, hs, sign);
    else
      rope_kernel<T, false><<<grid_cap(work), kThreads, 0, stream>>>((T*)out, (const T*)x, cosv, sinv, pos, tokens, seq, heads, dim, ts, hs, sign);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_swiglu_fwd(int dtype, void* out, const void* x, int64_t rows, int64_t h, cudaStream_t stream) {
  return b200_swiglu_fwd_rows(dtype, out, x, rows, h, nullptr, 0, stream);
}

int b200_swiglu_bwd(int dtype, void* dx, const void* dy, const void* x, int64_t rows, int64_t h, cudaStream_t stream) {
  return b200_swiglu_bwd_rows(dtype, dx, dy, x, rows, h, nullptr, 0, stream);
}

int b200_swiglu_fwd_rows(int dtype, void* out, const void* x, int64_t rows, int64_t h, const int* row_counts, int n_counts,
                         cudaStream_t stream) {
  if (rows == 0 || h == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    if (h % Vec16<T>::N != 0 || !aligned16((const T*)x) || !aligned16((T*)out)) return (int)cudaErrorNotSupported;
    const unsigned chunks = (unsigned)cdiv(h / Vec16<T>::N, (int64_t)kSwThreads * kSwU);
    if (rows > 2147483647ll || chunks > 65535u) return (int)cudaErrorNotSupported;
    swiglu_fwd_kernel<T><<<dim3((unsigned)rows, chunks), kSwThreads, 0, stream>>>((T*)out, (const T*)x, rows, h, row_counts, n_counts);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_swiglu_bwd_rows(int dtype, void* dx, const void* dy, const void* x, int64_t rows, int64_t h, const int* row_counts,
                         int n_counts, cudaStream_t stream) {
  if (rows == 0 || h == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    if (h % Vec16<T>::N != 0 || !aligned16((const T*)x) || !aligned16((T*)dx) || !aligned16((const T*)dy))
      return (int)cudaErrorNotSupported;
    const unsigned chunks = (unsigned)cdiv(h / Vec16<T>::N, (int64_t)kSwThreads * kSwU);
    if (rows > 2147483647ll || chunks > 65535u) return (int)cudaErrorNotSupported;
    swiglu_bwd_kernel<T><<<dim3((unsigned)rows, chunks), kSwThreads, 0, stream>>>((T*)dx, (const T*)dy, (const T*)x, rows, h, row_counts, n_counts);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_silu_mul_fwd(int dtype, void* out, const void* gate, const void* up, int64_t n, cudaStream_t stream) {
  if (n == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    if (!aligned16((const T*)gate) || !aligned16((const T*)up) || !aligned16((T*)out)) return (int)cudaErrorNotSupported;
    silu_mul_fwd_kernel<T><<<grid_cap(n / Vec16<T>::N + 1), kThreads, 0, stream>>>((T*)out, (const T*)gate, (const T*)up, n);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_silu_mul_bwd(int dtype, void* dgate, void* dup, const void* dy, const void* gate, const void* up, int64_t n,
                      cudaStream_t stream) {
  if (n == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    if (!aligned16((const T*)gate) || !aligned16((const T*)up) || !aligned16((const T*)dy) || !aligned16((T*)dgate) ||
        !aligned16((T*)dup))
      return (int)cudaErrorNotSupported;
    silu_mul_bwd_kernel<T><<<grid_cap(n / Vec16<T>::N + 1), kThreads, 0, stream>>>((T*)dgate, (T*)dup, (const T*)dy, (const T*)gate, (const T*)up, n);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_embedding_fwd(int dtype, void* out, const void* weight, const int64_t* idx, int64_t n, int64_t dim,
                       int64_t vocab, cudaStream_t stream) {
  if (n == 0 || dim == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    if (dim % Vec16<T>::N != 0 || !aligned16((const T*)weight) || !aligned16((T*)out)) return (int)cudaErrorNotSupported;
    embedding_fwd_kernel<T><<<grid_cap(n * dim / Vec16<T>::N), kThreads, 0, stream>>>((T*)out, (const T*)weight, idx, n, dim, vocab);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_embedding_bwd_atomic(int dtype, float* gw, const void* go, const int64_t* idx, int64_t n, int64_t dim,
                              int64_t vocab, int64_t padding_idx, cudaStream_t stream) {
  if (n == 0 || dim == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    embedding_bwd_atomic_kernel<T><<<grid_cap(n * dim), kThreads, 0, stream>>>(gw, (const T*)go, idx, n, dim, vocab, padding_idx);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_embedding_bwd_sorted(int dtype, void* gw, const void* go, const int64_t* sidx, const int64_t* perm, int64_t n,
                              int64_t dim, int64_t vocab, int64_t padding_idx, cudaStream_t stream) {
  if (n == 0 || dim == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    dim3 grid((unsigned)n, (unsigned)std::min<int64_t>(cdiv(dim, 128), 8));
    embedding_bwd_sorted_kernel<T><<<grid, 128, 0, stream>>>((T*)gw, (const T*)go, sidx, perm, n, dim, vocab, padding_idx);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_dropout_fwd(int dtype, void* out, uint8_t* mask, const void* x, int64_t n, float p, b200_philox_t rng,
                     cudaStream_t stream) {
  if (n == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    dropout_fwd_kernel<T><<<grid_cap(cdiv(n, 4)), kThreads, 0, stream>>>((T*)out, mask, (const T*)x, n, p, rng);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_dropout_bwd(int dtype, void* dx, const void* dy, const uint8_t* mask, int64_t n, float scale,
                     cudaStream_t stream) {
  if (n == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    dropout_bwd_kernel<T><<<grid_cap(n), kThreads, 0, stream>>>((T*)dx, (const T*)dy, mask, n, scale);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_uniform(int dtype, void* out, int64_t n, double lo, double hi, b200_philox_t rng, cudaStream_t s) {
  if (n == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    random_fill_kernel<T, false><<<grid_cap(cdiv(n, 4)), kThreads, 0, s>>>((T*)out, n, (float)lo, (float)hi, rng);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

int b200_normal(int dtype, void* out, int64_t n, double mean, double std, b200_philox_t rng, cudaStream_t s) {
  if (n == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    random_fill_kernel<T, true><<<grid_cap(cdiv(n, 4)), kThreads, 0, s>>>((T*)out, n, (float)mean, (float)std, rng);
    B200K_LAUNCH_RET();
  })
  return (int)cudaErrorNotSupported;
}

}  // extern "C"
