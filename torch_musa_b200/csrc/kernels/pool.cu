// 2-D pooling over [N, H, W, C] activations (channels-last; a contiguous NCHW tensor is the same layout with
// C = 1 and N * C images): max pooling with the argmax plane index, its backward in gather form (every input pixel
// visits the windows that cover it: deterministic, no atomics), average pooling and its backward.  Threads run
// along C, so every access is coalesced; fp32 arithmetic for the 16-bit types.
// Parity: reference torch_musa/csrc/aten/ops/Pool.cpp (vendor-library pooling).
#include "common.cuh"

namespace b200k {
namespace {

constexpr int kPoolThreads = 256;

struct PoolGeom {
  int64_t N, H, W, C, Ho, Wo;
  int kh, kw, sh, sw, ph, pw, dh, dw;
};

inline unsigned pool_blocks(int64_t n) { return (unsigned)std::min<int64_t>(cdiv(std::max<int64_t>(n, 1), kPoolThreads), 2147483647ll); }

template <typename T>
__global__ void __launch_bounds__(kPoolThreads) maxpool_fwd_kernel(T* __restrict__ out, int64_t* __restrict__ idx,
                                                                   const T* __restrict__ in, PoolGeom g) {
  const int64_t total = g.N * g.Ho * g.Wo * g.C;
  for (int64_t t = (int64_t)blockIdx.x * kPoolThreads + threadIdx.x; t < total; t += (int64_t)gridDim.x * kPoolThreads) {
    const int64_t c = t % g.C, wo = (t / g.C) % g.Wo, ho = (t / (g.C * g.Wo)) % g.Ho, n = t / (g.C * g.Wo * g.Ho);
    float best = -INFINITY;
    int64_t where = -1;
    for (int r = 0; r < g.kh; ++r) {
      const int64_t h = ho * g.sh - g.ph + (int64_t)r * g.dh;
      if (h < 0 || h >= g.H) continue;
      for (int s = 0; s < g.kw; ++s) {
        const int64_t w = wo * g.sw - g.pw + (int64_t)s * g.dw;
        if (w < 0 || w >= g.W) continue;
        const float v = ToF<T>::to(in[((n * g.H + h) * g.W + w) * g.C + c]);
        if (v > best || v != v || where < 0) {      // NaN propagates; the first maximum wins ties
          if (!(best != best)) { best = v; where = h * g.W + w; }
        }
      }
    }
    out[t] = ToF<T>::from(best);
    if (idx) idx[t] = where < 0 ? 0 : where;
  }
}

template <typename T>
__global__ void __launch_bounds__(kPoolThreads) maxpool_bwd_kernel(T* __restrict__ gin, const T* __restrict__ gout,
                                                                   const int64_t* __restrict__ idx, PoolGeom g) {
  const int64_t total = g.N * g.H * g.W * g.C;
  for (int64_t t = (int64_t)blockIdx.x * kPoolThreads + threadIdx.x; t < total; t += (int64_t)gridDim.x * kPoolThreads) {
    const int64_t c = t % g.C, w = (t / g.C) % g.W, h = (t / (g.C * g.W)) % g.H, n = t / (g.C * g.W * g.H);
    const int64_t me = h * g.W + w;
    // output rows / columns whose window can contain (h, w)
    const int64_t span_h = (int64_t)(g.kh - 1) * g.dh, span_w = (int64_t)(g.kw - 1) * g.dw;
    int64_t ho0 = (h + g.ph - span_h + g.sh - 1) / g.sh, ho1 = (h + g.ph) / g.sh;
    int64_t wo0 = (w + g.pw - span_w + g.sw - 1) / g.sw, wo1 = (w + g.pw) / g.sw;
    if (h + g.ph - span_h < 0) ho0 = 0;
    if (w + g.pw - span_w < 0) wo0 = 0;
    ho1 = min(ho1, g.Ho - 1);
    wo1 = min(wo1, g.Wo - 1);
    float acc = 0.f;
    for (int64_t ho = ho0; ho <= ho1; ++ho)
      for (int64_t wo = wo0; wo <= wo1; ++wo) {
        const int64_t o = ((n * g.Ho + ho) * g.Wo + wo) * g.C + c;
        if (idx[o] == me) acc += ToF<T>::to(gout[o]);
      }
    gin[t] = ToF<T>::from(acc);
  }
}

// ---- 16-bit types with C % 8 == 0 and fewer than 2^31 pixels: one thread owns 8 channels of a pixel (16-byte
// accesses, 32-bit index arithmetic).
template <typename T>
__global__ void __launch_bounds__(kPoolThreads) maxpool_fwd_vec_kernel(T* __restrict__ out, int64_t* __restrict__ idx,
                                                                       const T* __restrict__ in, PoolGeom g) {
  const int cv = (int)(g.C / 8), H = (int)g.H, W = (int)g.W, Ho = (int)g.Ho, Wo = (int)g.Wo;
  const long long total = (long long)g.N * Ho * Wo * cv;
  for (long long t = (long long)blockIdx.x * kPoolThreads + threadIdx.x; t < total; t += (long long)gridDim.x * kPoolThreads) {
    const int c8 = (int)(t % cv);
    const unsigned pix = (unsigned)(t / cv);
    const int wo = pix % Wo, ho = (pix / Wo) % Ho, n = pix / (Wo * Ho);
    float best[8];
    int where[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) { best[e] = -INFINITY; where[e] = -1; }
    for (int r = 0; r < g.kh; ++r) {
      const int h = ho * g.sh - g.ph + r * g.dh;
      if (h < 0 || h >= H) continue;
      for (int s = 0; s < g.kw; ++s) {
        const int w = wo * g.sw - g.pw + s * g.dw;
        if (w < 0 || w >= W) continue;
        const Vec16<T> v = ld16(in + (((long long)n * H + h) * W + w) * g.C + c8 * 8);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float f = ToF<T>::to(v.v[e]);
          if ((f > best[e] || f != f || where[e] < 0) && !(best[e] != best[e])) { best[e] = f; where[e] = h * W + w; }
        }
      }
    }
    Vec16<T> o;
#pragma unroll
    for (int e = 0; e < 8; ++e) o.v[e] = ToF<T>::from(best[e]);
    const long long off = (long long)pix * g.C + c8 * 8;
    st16(out + off, o);
    if (idx) {
#pragma unroll
      for (int e = 0; e < 8; e += 2) {
        longlong2 w2 = make_longlong2(where[e] < 0 ? 0 : where[e], where[e + 1] < 0 ? 0 : where[e + 1]);
        *reinterpret_cast<longlong2*>(idx + off + e) = w2;
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kPoolThreads) maxpool_bwd_vec_kernel(T* __restrict__ gin, const T* __restrict__ gout,
                                                                       const int64_t* __restrict__ idx, PoolGeom g) {
  const int cv = (int)(g.C / 8), H = (int)g.H, W = (int)g.W, Ho = (int)g.Ho, Wo = (int)g.Wo;
  const long long total = (long long)g.N * H * W * cv;
  const int span_h = (g.kh - 1) * g.dh, span_w = (g.kw - 1) * g.dw;
  for (long long t = (long long)blockIdx.x * kPoolThreads + threadIdx.x; t < total; t += (long long)gridDim.x * kPoolThreads) {
    const int c8 = (int)(t % cv);
    const unsigned pix = (unsigned)(t / cv);
    const int w = pix % W, h = (pix / W) % H, n = pix / (W * H);
    const long long me = (long long)h * W + w;
    int ho0 = h + g.ph - span_h < 0 ? 0 : (h + g.ph - span_h + g.sh - 1) / g.sh;
    int wo0 = w + g.pw - span_w < 0 ? 0 : (w + g.pw - span_w + g.sw - 1) / g.sw;
    const int ho1 = min((h + g.ph) / g.sh, Ho - 1), wo1 = min((w + g.pw) / g.sw, Wo - 1);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int ho = ho0; ho <= ho1; ++ho)
      for (int wo = wo0; wo <= wo1; ++wo) {
        const long long o = (((long long)n * Ho + ho) * Wo + wo) * g.C + c8 * 8;
        const Vec16<T> gv = ld16(gout + o);
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          const longlong2 i2 = *reinterpret_cast<const longlong2*>(idx + o + e);
          if (i2.x == me) acc[e] += ToF<T>::to(gv.v[e]);
          if (i2.y == me) acc[e + 1] += ToF<T>::to(gv.v[e + 1]);
        }
      }
    Vec16<T> r;
#pragma unroll
    for (int e = 0; e < 8; ++e) r.v[e] = ToF<T>::from(acc[e]);
    st16(gin + (long long)pix * g.C + c8 * 8, r);
  }
}

inline bool pool_vec_ok(const PoolGeom& g, int dtype, const void* a, const void* b, const void* idx) {
  if (dtype != B200_BF16 && dtype != B200_F16) return false;
  if (g.C % 8 != 0) return false;
  if (g.N * g.H * g.W >= (1ll << 31) || g.N * g.Ho * g.Wo >= (1ll << 31) || g.H * g.W >= (1ll << 31)) return false;
  return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(idx)) & 15) == 0;
}

// divisor: 0 = window size (count_include_pad), -1 = valid elements only, > 0 = fixed override
template <typename T>
__global__ void __launch_bounds__(kPoolThreads) avgpool_fwd_kernel(T* __restrict__ out, const T* __restrict__ in, PoolGeom g,
                                                                   int divisor) {
  const int64_t total = g.N * g.Ho * g.Wo * g.C;
  for (int64_t t = (int64_t)blockIdx.x * kPoolThreads + threadIdx.x; t < total; t += (int64_t)gridDim.x * kPoolThreads) {
    const int64_t c = t % g.C, wo = (t / g.C) % g.Wo, ho = (t / (g.C * g.Wo)) % g.Ho, n = t / (g.C * g.Wo * g.Ho);
    const int64_t h0 = ho * g.sh - g.ph, w0 = wo * g.sw - g.pw;
    const int64_t h1 = min(h0 + g.kh, g.H + g.ph), w1 = min(w0 + g.kw, g.W + g.pw);
    const int64_t pool = (h1 - h0) * (w1 - w0);             // window clipped to the padded extent
    const int64_t hs = max(h0, (int64_t)0), ws = max(w0, (int64_t)0), he = min(h1, g.H), we = min(w1, g.W);
    float acc = 0.f;
    for (int64_t h = hs; h < he; ++h)
      for (int64_t w = ws; w < we; ++w) acc += ToF<T>::to(in[((n * g.H + h) * g.W + w) * g.C + c]);
    const float div = divisor > 0 ? (float)divisor : (divisor == 0 ? (float)pool : (float)max((he - hs) * (we - ws), (int64_t)1));
    out[t] = ToF<T>::from(acc / div);
  }
}

template <typename T>
__global__ void __launch_bounds__(kPoolThreads) avgpool_bwd_kernel(T* __restrict__ gin, const T* __restrict__ gout, PoolGeom g,
                                                                   int divisor) {
  const int64_t total = g.N * g.H * g.W * g.C;
  for (int64_t t = (int64_t)blockIdx.x * kPoolThreads + threadIdx.x; t < total; t += (int64_t)gridDim.x * kPoolThreads) {
    const int64_t c = t % g.C, w = (t / g.C) % g.W, h = (t / (g.C * g.W)) % g.H, n = t / (g.C * g.W * g.H);
    int64_t ho0 = (h + g.ph - (g.kh - 1) + g.sh - 1) / g.sh, ho1 = (h + g.ph) / g.sh;
    int64_t wo0 = (w + g.pw - (g.kw - 1) + g.sw - 1) / g.sw, wo1 = (w + g.pw) / g.sw;
    if (h + g.ph - (g.kh - 1) < 0) ho0 = 0;
    if (w + g.pw - (g.kw - 1) < 0) wo0 = 0;
    ho1 = min(ho1, g.Ho - 1);
    wo1 = min(wo1, g.Wo - 1);
    float acc = 0.f;
    for (int64_t ho = ho0; ho <= ho1; ++ho)
      for (int64_t wo = wo0; wo <= wo1; ++wo) {
        const int64_t h0 = ho * g.sh - g.ph, w0 = wo * g.sw - g.pw;
        const int64_t h1 = min(h0 + g.kh, g.H + g.ph), w1 = min(w0 + g.kw, g.W + g.pw);
        if (h < h0 || h >= h1 || w < w0 || w >= w1) continue;
        const int64_t pool = (h1 - h0) * (w1 - w0);
        const int64_t hs = max(h0, (int64_t)0), ws = max(w0, (int64_t)0), he = min(h1, g.H), we = min(w1, g.W);
        const float div = divisor > 0 ? (float)divisor : (divisor == 0 ? (float)pool : (float)max((he - hs) * (we - ws), (int64_t)1));
        acc += ToF<T>::to(gout[((n * g.Ho + ho) * g.Wo + wo) * g.C + c]) / div;
      }
    gin[t] = ToF<T>::from(acc);
  }
}

PoolGeom geom_of(const b200_pool_t* p) {
  PoolGeom g;
  g.N = p->N; g.H = p->H; g.W = p->W; g.C = p->C; g.Ho = p->Ho; g.Wo = p->Wo;
  g.kh = p->kh; g.kw = p->kw; g.sh = p->sh; g.sw = p->sw; g.ph = p->ph; g.pw = p->pw; g.dh = p->dh; g.dw = p->dw;
  return g;
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" {

int b200_maxpool2d_fwd(const b200_pool_t* p, int dtype, void* out, int64_t* idx, const void* in, cudaStream_t stream) {
  const PoolGeom g = geom_of(p);
  const int64_t n = g.N * g.Ho * g.Wo * g.C;
  if (n == 0) return 0;
  if (pool_vec_ok(g, dtype, out, in, idx)) {
    const int64_t nv = n / 8;
    if (dtype == B200_BF16)
      maxpool_fwd_vec_kernel<__nv_bfloat16><<<pool_blocks(nv), kPoolThreads, 0, stream>>>((__nv_bfloat16*)out, idx, (const __nv_bfloat16*)in, g);
    else
      maxpool_fwd_vec_kernel<__half><<<pool_blocks(nv), kPoolThreads, 0, stream>>>((__half*)out, idx, (const __half*)in, g);
    B200K_LAUNCH_RET();
  }
  B200K_DISPATCH_FLOAT(dtype, T, (maxpool_fwd_kernel<T><<<pool_blocks(n), kPoolThreads, 0, stream>>>((T*)out, idx, (const T*)in, g)));
  B200K_LAUNCH_RET();
}
int b200_maxpool2d_bwd(const b200_pool_t* p, int dtype, void* gin, const void* gout, const int64_t* idx, cudaStream_t stream) {
  const PoolGeom g = geom_of(p);
  const int64_t n = g.N * g.H * g.W * g.C;
  if (n == 0) return 0;
  if (pool_vec_ok(g, dtype, gin, gout, idx)) {
    const int64_t nv = n / 8;
    if (dtype == B200_BF16)
      maxpool_bwd_vec_kernel<__nv_bfloat16><<<pool_blocks(nv), kPoolThreads, 0, stream>>>((__nv_bfloat16*)gin, (const __nv_bfloat16*)gout, idx, g);
    else
      maxpool_bwd_vec_kernel<__half><<<pool_blocks(nv), kPoolThreads, 0, stream>>>((__half*)gin, (const __half*)gout, idx, g);
    B200K_LAUNCH_RET();
  }
  B200K_DISPATCH_FLOAT(dtype, T, (maxpool_bwd_kernel<T><<<pool_blocks(n), kPoolThreads, 0, stream>>>((T*)gin, (const T*)gout, idx, g)));
  B200K_LAUNCH_RET();
}
int b200_avgpool2d_fwd(const b200_pool_t* p, int dtype, void* out, const void* in, int divisor, cudaStream_t stream) {
  const PoolGeom g = geom_of(p);
  const int64_t n = g.N * g.Ho * g.Wo * g.C;
  if (n == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, (avgpool_fwd_kernel<T><<<pool_blocks(n), kPoolThreads, 0, stream>>>((T*)out, (const T*)in, g, divisor)));
  B200K_LAUNCH_RET();
}
int b200_avgpool2d_bwd(const b200_pool_t* p, int dtype, void* gin, const void* gout, int divisor, cudaStream_t stream) {
  const PoolGeom g = geom_of(p);
  const int64_t n = g.N * g.H * g.W * g.C;
  if (n == 0) return 0;
  B200K_DISPATCH_FLOAT(dtype, T, (avgpool_bwd_kernel<T><<<pool_blocks(n), kPoolThreads, 0, stream>>>((T*)gin, (const T*)gout, g, divisor)));
  B200K_LAUNCH_RET();
}

}  // extern "C"
