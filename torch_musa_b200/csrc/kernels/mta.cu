// multi_tensor_apply: one launch updates up to 128 tensors / 1184 chunks.  The
// tensor table travels in kernel-parameter space (sm_100 accepts 32 KB of
// parameters), so there is no metadata upload and the whole optimizer step of a
// ResNet-50 (161 tensors) is two launches.  Each CTA owns one chunk of one
// tensor; chunks are sized so the grid is a few waves of the 148 SMs.
// Functors: Adam/AdamW (+amsgrad, tensor lr, GradScaler-aware), SGD (momentum,
// nesterov, dampening), L2 norms (per tensor + global, two-stage deterministic),
// unscale-and-check, axpby, LAMB stages, and the GradScaler update.
// Parity: reference torch_musa/csrc/extension/common/multi_tensor_apply.muh:16-27,
// FusedAdam.mu:57-137,348-472, aten/ops/musa/FusedSgdKernel.mu:15-145,
// apex/multi_tensor_l2norm_kernel.mu:195-342, apex/multi_tensor_lamb.mu, aten/ops/musa/Amp.mu:22-44.
#include "common.cuh"

#include <algorithm>
#include <vector>

namespace b200k {
namespace {

constexpr int kMaxTensors = 128;
constexpr int kMaxBlocks = kSMs * 8;  // 1184
constexpr int kThreads = 512;
constexpr int kMinChunk = 65536;
constexpr int kNormSlots = 320;  // partial-sum slots per tensor in the L2-norm scratch

template <int DEPTH>
struct Meta {
  void* addr[DEPTH][kMaxTensors];
  int64_t numel[kMaxTensors];
  int32_t block_chunk[kMaxBlocks];
  uint16_t block_tensor[kMaxBlocks];
  int32_t gidx[kMaxTensors];  // position of the tensor in the caller's list
  int32_t start_tensor;
  int32_t n_tensors;
  int64_t chunk;
};

template <int DEPTH, typename F, typename... A>
__global__ void __launch_bounds__(kThreads) mta_kernel(const __grid_constant__ Meta<DEPTH> meta, F f, A... args) {
  const int t = meta.block_tensor[blockIdx.x];
  const int64_t c = meta.block_chunk[blockIdx.x];
  const int64_t begin = c * meta.chunk;
  int64_t n = meta.numel[t] - begin;
  if (n > meta.chunk) n = meta.chunk;
  f(meta, t, begin, n, args...);
}

// Walks the tensor lists, packs launches.
template <int DEPTH, typename F, typename... A>
int mta_launch(int n_tensors, void* const* const* lists, const int64_t* numels, int64_t chunk, cudaStream_t stream, F f,
               A... args) {
  Meta<DEPTH> meta;
  meta.chunk = chunk;
  int nt = 0, nb = 0;
  meta.start_tensor = 0;
  auto flush = [&](int next_start) -> int {
    if (nb > 0) {
      meta.n_tensors = nt;
      mta_kernel<DEPTH, F, A...><<<nb, kThreads, 0, stream>>>(meta, f, args...);
      note_launch();
      cudaError_t e = cudaGetLastError();
      if (e != cudaSuccess) return (int)e;
    }
    nt = 0;
    nb = 0;
    meta.start_tensor = next_start;
    return 0;
  };
  for (int t = 0; t < n_tensors; ++t) {
    if (numels[t] == 0) continue;
    int64_t chunks = cdiv(numels[t], chunk);
    int64_t done = 0;
    while (done < chunks) {
      if (nt == kMaxTensors || nb == kMaxBlocks) {
        int e = flush(t);
        if (e) return e;
      }
      // (re)open tensor t in this launch
      if (nt == 0) meta.start_tensor = t;
      int slot = nt++;
      for (int d = 0; d < DEPTH; ++d) meta.addr[d][slot] = lists[d] ? lists[d][t] : nullptr;
      meta.numel[slot] = numels[t];
      meta.gidx[slot] = t;
      while (done < chunks && nb < kMaxBlocks) {
        meta.block_tensor[nb] = (uint16_t)slot;
        meta.block_chunk[nb] = (int32_t)done;
        ++nb;
        ++done;
      }
      if (done < chunks) {
        // launch is full of blocks but the tensor continues: flush and reopen it
        int e = flush(t);
        if (e) return e;
      }
    }
  }
  return flush(n_tensors);
}

inline int64_t pick_chunk(int n_tensors, const int64_t* numels, int64_t max_slots = 0) {
  int64_t total = 0, mx = 0;
  for (int i = 0; i < n_tensors; ++i) { total += numels[i]; mx = std::max(mx, numels[i]); }
  // aim for ~4 waves of CTAs over the whole list, never below 64K elements per CTA
  int64_t c = std::max<int64_t>(kMinChunk, cdiv(total, (int64_t)kMaxBlocks * 4));
  if (max_slots > 0) c = std::max<int64_t>(c, cdiv(mx, max_slots));
  return cdiv(c, 4096) * 4096;
}

// 4-element packets: 16 B for fp32, 8 B for 16-bit types
template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&o)[4]) {
  if constexpr (sizeof(T) == 4) {
    float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  } else {
    uint2 raw = *reinterpret_cast<const uint2*>(p);
    const T* t = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) o[k] = ToF<T>::to(t[k]);
  }
}
template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&o)[4]) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
  } else {
    uint2 raw;
    T* t = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int k = 0; k < 4; ++k) t[k] = ToF<T>::from(o[k]);
    *reinterpret_cast<uint2*>(p) = raw;
  }
}
__device__ __forceinline__ bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---------------------------------------------------------------- Adam / AdamW
template <typename TP, typename TG, typename TS>
struct AdamFunctor {
  __device__ void operator()(const Meta<6>& m, int t, int64_t begin, int64_t n, b200_adam_args_t a) const {
    if (a.found_inf && *a.found_inf != 0.f) return;
    TP* p = (TP*)m.addr[0][t] + begin;
    TG* g = (TG*)m.addr[1][t] + begin;
    TS* ea = (TS*)m.addr[2][t] + begin;
    TS* es = (TS*)m.addr[3][t] + begin;
    TS* mx = a.amsgrad ? (TS*)m.addr[4][t] + begin : nullptr;
    const float step = *(const float*)m.addr[5][t];
    const float lr = a.lr_ptr ? *a.lr_ptr : a.lr;
    const float inv_scale = a.grad_scale ? 1.f / *a.grad_scale : 1.f;
    const float bc1 = 1.f - powf(a.beta1, step);
    const float bc2s = sqrtf(1.f - powf(a.beta2, step));
    const float step_size = lr / bc1;
    auto upd = [&](float& pf, float& gf, float& mf, float& vf, float& mxf) {
      if (a.grad_scale) gf *= inv_scale;
      float ge = a.maximize ? -gf : gf;
      if (a.adamw) pf -= lr * a.weight_decay * pf; else ge += a.weight_decay * pf;
      mf = a.beta1 * mf + (1.f - a.beta1) * ge;
      vf = a.beta2 * vf + (1.f - a.beta2) * ge * ge;
      float denom;
      if (mx) {
        mxf = fmaxf(mxf, vf);
        denom = sqrtf(mxf) / bc2s + a.eps;
      } else {
        denom = sqrtf(vf) / bc2s + a.eps;
      }
      pf -= step_size * mf / denom;
    };
    const bool vec = al16(p) && al16(g) && al16(ea) && al16(es) && (!mx || al16(mx));
    const int64_t n4 = vec ? n / 4 : 0;
    // 4 independent 4-element packets per thread per trip: all loads are issued before any math so that
    // 16 x 16 B are in flight per thread (the step is pure HBM streaming: 16 B read + 12 B written per element)
    constexpr int ILP = 4;
    for (int64_t q0 = threadIdx.x; q0 < n4; q0 += (int64_t)kThreads * ILP) {
      float pf[ILP][4], gf[ILP][4], mf[ILP][4], vf[ILP][4], xf[ILP][4];
#pragma unroll
      for (int u = 0; u < ILP; ++u) {
        const int64_t q = q0 + (int64_t)u * kThreads;
        if (q < n4) {
          const int64_t i = q * 4;
          load4(p + i, pf[u]); load4(g + i, gf[u]); load4(ea + i, mf[u]); load4(es + i, vf[u]);
          if (mx) load4(mx + i, xf[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < ILP; ++u) {
        const int64_t q = q0 + (int64_t)u * kThreads;
        if (q < n4) {
          const int64_t i = q * 4;
          if (!mx) { xf[u][0] = xf[u][1] = xf[u][2] = xf[u][3] = 0.f; }
#pragma unroll
          for (int k = 0; k < 4; ++k) upd(pf[u][k], gf[u][k], mf[u][k], vf[u][k], xf[u][k]);
          store4(p + i, pf[u]); store4(ea + i, mf[u]); store4(es + i, vf[u]);
          if (mx) store4(mx + i, xf[u]);
          if (a.grad_scale) store4(g + i, gf[u]);
        }
      }
    }
    for (int64_t i = n4 * 4 + threadIdx.x; i < n; i += kThreads) {
      float pf = ToF<TP>::to(p[i]), gf = ToF<TG>::to(g[i]), mf = ToF<TS>::to(ea[i]), vf = ToF<TS>::to(es[i]);
      float xf = mx ? ToF<TS>::to(mx[i]) : 0.f;
      upd(pf, gf, mf, vf, xf);
      p[i] = ToF<TP>::from(pf); ea[i] = ToF<TS>::from(mf); es[i] = ToF<TS>::from(vf);
      if (mx) mx[i] = ToF<TS>::from(xf);
      if (a.grad_scale) g[i] = ToF<TG>::from(gf);
    }
  }
};

// ---------------------------------------------------------------- SGD
template <typename TP, typename TG>
struct SgdFunctor {
  __device__ void operator()(const Meta<3>& m, int t, int64_t begin, int64_t n, b200_sgd_args_t a) const {
    if (a.found_inf && *a.found_inf != 0.f) return;
    TP* p = (TP*)m.addr[0][t] + begin;
    TG* g = (TG*)m.addr[1][t] + begin;
    TP* buf = m.addr[2][t] ? (TP*)m.addr[2][t] + begin : nullptr;
    const float lr = a.lr_ptr ? *a.lr_ptr : a.lr;
    const float inv_scale = a.grad_scale ? 1.f / *a.grad_scale : 1.f;
    auto upd = [&](float& pf, float& gf, float& bf) {
      if (a.grad_scale) gf *= inv_scale;
      float ge = a.maximize ? -gf : gf;
      if (a.weight_decay != 0.f) ge += a.weight_decay * pf;
      if (buf) {
        bf = a.first_step ? ge : a.momentum * bf + (1.f - a.dampening) * ge;
        ge = a.nesterov ? ge + a.momentum * bf : bf;
      }
      pf -= lr * ge;
    };
    const bool vec = al16(p) && al16(g) && (!buf || al16(buf));
    const int64_t n4 = vec ? n / 4 : 0;
    for (int64_t q = threadIdx.x; q < n4; q += kThreads) {
      const int64_t i = q * 4;
      float pf[4], gf[4], bf[4] = {0.f, 0.f, 0.f, 0.f};
      load4(p + i, pf); load4(g + i, gf);
      if (buf && !a.first_step) load4(buf + i, bf);
#pragma unroll
      for (int k = 0; k < 4; ++k) upd(pf[k], gf[k], bf[k]);
      store4(p + i, pf);
      if (buf) store4(buf + i, bf);
      if (a.grad_scale) store4(g + i, gf);
    }
    for (int64_t i = n4 * 4 + threadIdx.x; i < n; i += kThreads) {
      float pf = ToF<TP>::to(p[i]), gf = ToF<TG>::to(g[i]), bf = (buf && !a.first_step) ? ToF<TP>::to(buf[i]) : 0.f;
      upd(pf, gf, bf);
      p[i] = ToF<TP>::from(pf);
      if (buf) buf[i] = ToF<TP>::from(bf);
      if (a.grad_scale) g[i] = ToF<TG>::from(gf);
    }
  }
};

// ---------------------------------------------------------------- L2 norm
template <typename T>
struct L2Functor {
  __device__ void operator()(const Meta<1>& m, int t, int64_t begin, int64_t n, float* partial) const {
    __shared__ float sh[32];
    const T* x = (const T*)m.addr[0][t] + begin;
    float acc = 0.f;
    const int64_t n4 = al16(x) ? n / 4 : 0;
    for (int64_t q = threadIdx.x; q < n4; q += kThreads) {
      float v[4];
      load4(x + q * 4, v);
      acc += v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
    }
    for (int64_t i = n4 * 4 + threadIdx.x; i < n; i += kThreads) {
      float v = ToF<T>::to(x[i]);
      acc += v * v;
    }
    acc = block_sum(acc, sh);
    if (threadIdx.x == 0)
      partial[(int64_t)m.gidx[t] * kNormSlots + m.block_chunk[blockIdx.x]] = acc;
  }
};

__global__ void l2_cleanup_kernel(float* __restrict__ per_tensor, const float* __restrict__ partial,
                                  const int64_t* __restrict__ nchunks_or_null, int64_t chunk, Meta<1> meta) {
  // one CTA per tensor of the batch
  __shared__ float sh[32];
  const int t = blockIdx.x;
  const int64_t chunks = (meta.numel[t] + chunk - 1) / chunk;
  float acc = 0.f;
  for (int64_t i = threadIdx.x; i < chunks; i += blockDim.x) acc += partial[(int64_t)(meta.start_tensor + t) * kNormSlots + i];
  acc = block_sum(acc, sh);
  if (threadIdx.x == 0) per_tensor[meta.start_tensor + t] = sqrtf(acc);
}

__global__ void l2_total_kernel(float* __restrict__ total, const float* __restrict__ per_tensor, int n) {
  __shared__ float sh[32];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) acc += per_tensor[i] * per_tensor[i];
  acc = block_sum(acc, sh);
  if (threadIdx.x == 0) *total = sqrtf(acc);
}

// ---------------------------------------------------------------- scale + finite check
template <typename T>
struct ScaleFunctor {
  __device__ void operator()(const Meta<1>& m, int t, int64_t begin, int64_t n, const float* inv_scale_ptr,
                             float host_scale, float* found_inf) const {
    T* x = (T*)m.addr[0][t] + begin;
    const float s = inv_scale_ptr ? *inv_scale_ptr : host_scale;
    bool bad = false;
    for (int64_t i = threadIdx.x; i < n; i += kThreads) {
      float v = ToF<T>::to(x[i]);
      if (!isfinite(v)) bad = true;
      x[i] = ToF<T>::from(s == 1.f ? v : v * s);
    }
    if (bad && found_inf) *found_inf = 1.f;
  }
};

template <typename T>
struct AxpbyFunctor {
  __device__ void operator()(const Meta<3>& m, int t, int64_t begin, int64_t n, float a, float b) const {
    T* o = (T*)m.addr[0][t] + begin;
    const T* x = (const T*)m.addr[1][t] + begin;
    const T* y = m.addr[2][t] ? (const T*)m.addr[2][t] + begin : nullptr;
    for (int64_t i = threadIdx.x; i < n; i += kThreads) {
      float v = a * ToF<T>::to(x[i]);
      if (y) v += b * ToF<T>::to(y[i]);
      o[i] = ToF<T>::from(v);
    }
  }
};

// ---------------------------------------------------------------- generic pointwise over tensor lists (_foreach_*)
// out = f(a[, b[, c]]); packets of four elements when every pointer of the chunk is suitably aligned
template <typename T>
struct ForeachFunctor {
  __device__ __forceinline__ static float apply(int op, float a, float b, float c, float s0, float s1) {
    switch (op) {
      case B200_FE_ADD_SCALAR: return a + s0;
      case B200_FE_MUL_SCALAR: return a * s0;
      case B200_FE_DIV_SCALAR: return a / s0;
      case B200_FE_ADD: return a + s0 * b;
      case B200_FE_MUL: return a * b;
      case B200_FE_DIV: return a / b;
      case B200_FE_ADDCMUL: return a + s0 * b * c;
      case B200_FE_ADDCDIV: return a + s0 * b / c;
      case B200_FE_LERP: return a + s0 * (b - a);
      case B200_FE_SQRT: return sqrtf(a);
      case B200_FE_NEG: return -a;
      case B200_FE_RECIPROCAL: return 1.f / a;
      case B200_FE_ABS: return fabsf(a);
      case B200_FE_MAXIMUM: return (a != a || b != b) ? NAN : fmaxf(a, b);
      case B200_FE_MINIMUM: return (a != a || b != b) ? NAN : fminf(a, b);
      case B200_FE_CLAMP: return a != a ? a : fminf(fmaxf(a, s0), s1);
      case B200_FE_ZERO: return 0.f;
      default: return a;   // COPY
    }
  }
  __device__ void operator()(const Meta<4>& m, int t, int64_t begin, int64_t n, int op, float s0, float s1) const {
    T* o = (T*)m.addr[0][t] + begin;
    const T* a = (const T*)m.addr[1][t] + begin;
    const T* b = m.addr[2][t] ? (const T*)m.addr[2][t] + begin : nullptr;
    const T* c = m.addr[3][t] ? (const T*)m.addr[3][t] + begin : nullptr;
    constexpr uintptr_t kMask = sizeof(T) * 4 - 1;
    const bool vec = (((uintptr_t)o | (uintptr_t)a | (uintptr_t)(b ? b : a) | (uintptr_t)(c ? c : a)) & kMask) == 0;
    const int64_t n4 = vec ? n / 4 : 0;
    for (int64_t i = threadIdx.x; i < n4; i += kThreads) {
      float va[4], vb[4] = {0.f, 0.f, 0.f, 0.f}, vc[4] = {0.f, 0.f, 0.f, 0.f}, r[4];
      load4(a + i * 4, va);
      if (b) load4(b + i * 4, vb);
      if (c) load4(c + i * 4, vc);
#pragma unroll
      for (int k = 0; k < 4; ++k) r[k] = apply(op, va[k], vb[k], vc[k], s0, s1);
      store4(o + i * 4, r);
    }
    for (int64_t i = n4 * 4 + threadIdx.x; i < n; i += kThreads)
      o[i] = ToF<T>::from(apply(op, ToF<T>::to(a[i]), b ? ToF<T>::to(b[i]) : 0.f, c ? ToF<T>::to(c[i]) : 0.f, s0, s1));
  }
};

// ---------------------------------------------------------------- LAMB
// stage 1: moments + raw update u (written over the gradient copy in `upd`), stage 2: trust-ratio apply
template <typename T>
struct LambStage1 {
  __device__ void operator()(const Meta<5>& m, int t, int64_t begin, int64_t n, b200_lamb_args_t a) const {
    T* p = (T*)m.addr[0][t] + begin;
    const T* g = (const T*)m.addr[1][t] + begin;
    T* ea = (T*)m.addr[2][t] + begin;
    T* es = (T*)m.addr[3][t] + begin;
    float* u = (float*)m.addr[4][t] + begin;
    float clip = 1.f;
    if (a.global_grad_norm && a.max_grad_norm > 0.f) {
      float gn = *a.global_grad_norm;
      clip = gn > a.max_grad_norm ? gn / a.max_grad_norm : 1.f;
    }
    const float bc1 = a.bias_correction ? 1.f - powf(a.beta1, (float)a.step) : 1.f;
    const float bc2 = a.bias_correction ? 1.f - powf(a.beta2, (float)a.step) : 1.f;
    const float b3 = a.grad_averaging ? 1.f - a.beta1 : 1.f;
    for (int64_t i = threadIdx.x; i < n; i += kThreads) {
      float gf = ToF<T>::to(g[i]) / clip, pf = ToF<T>::to(p[i]);
      if (!a.adam_w_mode) gf += a.weight_decay * pf;
      float mf = a.beta1 * ToF<T>::to(ea[i]) + b3 * gf;
      float vf = a.beta2 * ToF<T>::to(es[i]) + (1.f - a.beta2) * gf * gf;
      ea[i] = ToF<T>::from(mf);
      es[i] = ToF<T>::from(vf);
      float upd = (mf / bc1) / (sqrtf(vf / bc2) + a.eps);
      if (a.adam_w_mode) upd += a.weight_decay * pf;
      u[i] = upd;
    }
  }
};

template <typename T>
struct LambStage2 {
  __device__ void operator()(const Meta<2>& m, int t, int64_t begin, int64_t n, b200_lamb_args_t a,
                             const float* pnorm, const float* unorm) const {
    T* p = (T*)m.addr[0][t] + begin;
    const float* u = (const float*)m.addr[1][t] + begin;
    const int gt = m.gidx[t];
    float ratio = 1.f;
    if (a.use_nvlamb || a.weight_decay != 0.f) {
      float pn = pnorm[gt], un = unorm[gt];
      ratio = (pn != 0.f && un != 0.f) ? pn / un : 1.f;
    }
    const float lr = a.lr * ratio;
    for (int64_t i = threadIdx.x; i < n; i += kThreads) p[i] = ToF<T>::from(ToF<T>::to(p[i]) - lr * u[i]);
  }
};

__global__ void amp_update_scale_kernel(float* scale, int* tracker, const float* found_inf, float growth,
                                        float backoff, int interval) {
  if (*found_inf != 0.f) {
    *scale = *scale * backoff;
    *tracker = 0;
  } else {
    int ok = *tracker + 1;
    if (ok == interval) {
      float ns = *scale * growth;
      if (isfinite(ns)) *scale = ns;
      *tracker = 0;
    } else {
      *tracker = ok;
    }
  }
}

template <typename T>
int l2norm_impl(int n, void* const* tensors, const int64_t* numels, float* out_total, float* out_per_tensor,
                float* scratch, cudaStream_t stream) {
  float* partial = scratch;
  float* per = out_per_tensor ? out_per_tensor : scratch + (size_t)n * kNormSlots;
  int64_t chunk = pick_chunk(n, numels, kNormSlots);
  void* const* lists[1] = {tensors};
  int e = mta_launch<1>(n, lists, numels, chunk, stream, L2Functor<T>(), partial);
  if (e) return e;
  // cleanup per batch of kMaxTensors
  for (int s = 0; s < n; s += kMaxTensors) {
    Meta<1> meta;
    int cnt = std::min(kMaxTensors, n - s);
    meta.start_tensor = s;
    meta.n_tensors = cnt;
    meta.chunk = chunk;
    for (int i = 0; i < cnt; ++i) meta.numel[i] = numels[s + i];
    l2_cleanup_kernel<<<cnt, 128, 0, stream>>>(per, partial, nullptr, chunk, meta);
    note_launch();
  }
  if (out_total) {
    l2_total_kernel<<<1, 256, 0, stream>>>(out_total, per, n);
    note_launch();
  }
  return (int)cudaGetLastError();
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" {

int b200_multi_tensor_adam(int n, int pd, int gd, int sd, void* const* params, void* const* grads,
                           void* const* exp_avg, void* const* exp_avg_sq, void* const* max_exp_avg_sq,
                           float* const* steps, const int64_t* numels, b200_adam_args_t args, cudaStream_t stream) {
  if (n == 0) return 0;
  void* const* lists[6] = {params, grads, exp_avg, exp_avg_sq, args.amsgrad ? max_exp_avg_sq : nullptr,
                           (void* const*)steps};
  int64_t chunk = pick_chunk(n, numels);
#define ADAM_GO(TP, TG, TS) return mta_launch<6>(n, lists, numels, chunk, stream, AdamFunctor<TP, TG, TS>(), args)
  if (pd == B200_F32 && gd == B200_F32 && sd == B200_F32) ADAM_GO(float, float, float);
  if (pd == B200_BF16 && gd == B200_BF16 && sd == B200_BF16) ADAM_GO(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  if (pd == B200_BF16 && gd == B200_BF16 && sd == B200_F32) ADAM_GO(__nv_bfloat16, __nv_bfloat16, float);
  if (pd == B200_F32 && gd == B200_BF16 && sd == B200_F32) ADAM_GO(float, __nv_bfloat16, float);
  if (pd == B200_BF16 && gd == B200_F32 && sd == B200_F32) ADAM_GO(__nv_bfloat16, float, float);
  if (pd == B200_F16 && gd == B200_F16 && sd == B200_F16) ADAM_GO(__half, __half, __half);
  if (pd == B200_F16 && gd == B200_F16 && sd == B200_F32) ADAM_GO(__half, __half, float);
  if (pd == B200_F32 && gd == B200_F16 && sd == B200_F32) ADAM_GO(float, __half, float);
#undef ADAM_GO
  return (int)cudaErrorNotSupported;
}

int b200_multi_tensor_sgd(int n, int pd, int gd, void* const* params, void* const* grads, void* const* bufs,
                          const int64_t* numels, b200_sgd_args_t args, cudaStream_t stream) {
  if (n == 0) return 0;
  void* const* lists[3] = {params, grads, bufs};
  int64_t chunk = pick_chunk(n, numels);
#define SGD_GO(TP, TG) return mta_launch<3>(n, lists, numels, chunk, stream, SgdFunctor<TP, TG>(), args)
  if (pd == B200_F32 && gd == B200_F32) SGD_GO(float, float);
  if (pd == B200_BF16 && gd == B200_BF16) SGD_GO(__nv_bfloat16, __nv_bfloat16);
  if (pd == B200_F16 && gd == B200_F16) SGD_GO(__half, __half);
  if (pd == B200_F32 && gd == B200_BF16) SGD_GO(float, __nv_bfloat16);
  if (pd == B200_F32 && gd == B200_F16) SGD_GO(float, __half);
#undef SGD_GO
  return (int)cudaErrorNotSupported;
}

size_t b200_multi_tensor_l2norm_scratch_floats(int n) { return (size_t)n * kNormSlots + (size_t)n + 8; }

int b200_multi_tensor_l2norm(int n, int dtype, void* const* tensors, const int64_t* numels, float* out_total,
                             float* out_per_tensor, float* scratch, cudaStream_t stream) {
  if (n == 0) {
    if (out_total) return (int)cudaMemsetAsync(out_total, 0, sizeof(float), stream);
    return 0;
  }
  B200K_DISPATCH_FLOAT(dtype, T, return l2norm_impl<T>(n, tensors, numels, out_total, out_per_tensor, scratch, stream));
  return (int)cudaErrorNotSupported;
}

int b200_multi_tensor_scale(int n, int dtype, void* const* tensors, const int64_t* numels, const float* inv_scale_ptr,
                            float host_scale, float* found_inf, cudaStream_t stream) {
  if (n == 0) return 0;
  void* const* lists[1] = {tensors};
  int64_t chunk = pick_chunk(n, numels);
  B200K_DISPATCH_FLOAT(dtype, T,
                       return mta_launch<1>(n, lists, numels, chunk, stream, ScaleFunctor<T>(), inv_scale_ptr,
                                            host_scale, found_inf));
  return (int)cudaErrorNotSupported;
}

int b200_multi_tensor_axpby(int n, int dtype, void* const* out, void* const* x, void* const* y, const int64_t* numels,
                            float a, float b, cudaStream_t stream) {
  if (n == 0) return 0;
  void* const* lists[3] = {out, x, y};
  int64_t chunk = pick_chunk(n, numels);
  B200K_DISPATCH_FLOAT(dtype, T, return mta_launch<3>(n, lists, numels, chunk, stream, AxpbyFunctor<T>(), a, b));
  return (int)cudaErrorNotSupported;
}

int b200_multi_tensor_pointwise(int op, int n, int dtype, void* const* out, void* const* a, void* const* b, void* const* c,
                                const int64_t* numels, float s0, float s1, cudaStream_t stream) {
  if (n == 0) return 0;
  void* const* lists[4] = {out, a, b, c};
  int64_t chunk = pick_chunk(n, numels);
  B200K_DISPATCH_FLOAT(dtype, T, return mta_launch<4>(n, lists, numels, chunk, stream, ForeachFunctor<T>(), op, s0, s1));
  return (int)cudaErrorNotSupported;
}

size_t b200_multi_tensor_lamb_scratch_floats(int n, const int64_t* numels) {
  size_t tot = 0;
  for (int i = 0; i < n; ++i) tot += (size_t)((numels[i] + 3) / 4 * 4);
  // updates + two l2norm scratches + two per-tensor norm arrays
  return tot + 2 * b200_multi_tensor_l2norm_scratch_floats(n) + 2 * (size_t)n + 16;
}

int b200_multi_tensor_lamb(int n, int dtype, void* const* params, void* const* grads, void* const* exp_avg,
                           void* const* exp_avg_sq, const int64_t* numels, b200_lamb_args_t args, float* scratch,
                           cudaStream_t stream) {
  if (n == 0) return 0;
  std::vector<void*> upd(n);
  size_t off = 0;
  for (int i = 0; i < n; ++i) { upd[i] = scratch + off; off += (size_t)((numels[i] + 3) / 4 * 4); }
  float* s1 = scratch + off;
  float* s2 = s1 + b200_multi_tensor_l2norm_scratch_floats(n);
  float* pnorm = s2 + b200_multi_tensor_l2norm_scratch_floats(n);
  float* unorm = pnorm + n;
  int64_t chunk = pick_chunk(n, numels);
  int e = 0;
  B200K_DISPATCH_FLOAT(dtype, T, {
    void* const* l5[5] = {params, grads, exp_avg, exp_avg_sq, upd.data()};
    e = mta_launch<5>(n, l5, numels, chunk, stream, LambStage1<T>(), args);
    if (e) return e;
    e = l2norm_impl<T>(n, params, numels, nullptr, pnorm, s1, stream);
    if (e) return e;
    e = l2norm_impl<float>(n, upd.data(), numels, nullptr, unorm, s2, stream);
    if (e) return e;
    void* const* l2[2] = {params, upd.data()};
    return mta_launch<2>(n, l2, numels, chunk, stream, LambStage2<T>(), args, (const float*)pnorm, (const float*)unorm);
  })
  return (int)cudaErrorNotSupported;
}

int b200_amp_update_scale(float* scale, int* growth_tracker, const float* found_inf, float growth, float backoff,
                          int growth_interval, cudaStream_t stream) {
  amp_update_scale_kernel<<<1, 1, 0, stream>>>(scale, growth_tracker, found_inf, growth, backoff, growth_interval);
  B200K_LAUNCH_RET();
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the multi-tensor L2 norm (declared in b200_no_alloc.h).
#include "b200_no_alloc.h"

namespace {

constexpr size_t kStaticScratchFloats = (size_t)B200_L2NORM_STATIC_MAX_TENSORS * (kNormSlots + 1) + 8;

// Lives in the library image on every device that loads it; in host code this name is only a handle
// for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) float g_l2norm_static_scratch[kStaticScratchFloats];

constexpr int kMaxStaticDevices = 64;
float* g_static_scratch_addr[kMaxStaticDevices] = {nullptr};

// Device address of the array on the current device (looked up once per device).
int static_scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxStaticDevices) return (int)cudaErrorInvalidDevice;
  if (!g_static_scratch_addr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_l2norm_static_scratch);
    if (e != cudaSuccess) return (int)e;
    g_static_scratch_addr[dev] = p;
  }
  *out = g_static_scratch_addr[dev];
  return 0;
}

}  // namespace

extern "C" int b200_multi_tensor_l2norm_static(int n, int dtype, void* const* tensors, const int64_t* numels,
                                               float* out_total, float* out_per_tensor, cudaStream_t stream) {
  if (n < 0 || n > B200_L2NORM_STATIC_MAX_TENSORS) return (int)cudaErrorInvalidValue;
  if (n == 0) {
    if (out_total) return (int)cudaMemsetAsync(out_total, 0, sizeof(float), stream);
    return 0;
  }
  float* scratch = nullptr;
  int e = static_scratch_for_current_device(&scratch);
  if (e) return e;
  B200K_DISPATCH_FLOAT(dtype, T,
                       return b200k::l2norm_impl<T>(n, tensors, numels, out_total, out_per_tensor, scratch, stream));
  return (int)cudaErrorNotSupported;
}
