// Single-query ("decode") attention over a static KV cache, head_dim 128.
//
// One CTA per (batch, query head), eight warps; warp w owns every eighth block of 32 keys in [0, *pos], the
// lanes split the 128 dimensions four each.  Per key: 4 FMAs + a warp sum for the score, online softmax in the
// log2 domain, 4 FMAs into the output slice; four keys are in flight per iteration.  The eight partial (max, sum,
// output) triples are merged through shared memory.  The visible length is read from device memory, so the
// kernel can sit inside a captured graph and follow the position counter without any host involvement.
// Memory-bound by design: K and V are read exactly once per query head (grouped-query heads re-read their
// shared KV head through L2).
// Parity: the reference has no decode kernel; it relies on the vendor SDPA (reference
// torch_musa/csrc/aten/ops/attention/mudnn/SDP.cpp).
#include "common.cuh"

namespace b200k {
namespace {

constexpr int DD = 128;
constexpr int kDecWarps = 8;

template <typename T>
__global__ void __launch_bounds__(kDecWarps * 32)
decode_attn_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ kc, const T* __restrict__ vc,
                   const long long* __restrict__ pos_ptr, int H, int Hkv, int max_len, float scale_log2) {
  __shared__ float sh_m[kDecWarps], sh_l[kDecWarps], sh_o[kDecWarps][DD];
  const int b = blockIdx.x / H, h = blockIdx.x - b * H;
  const int hk = h / (H / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long n_keys = *pos_ptr + 1;
  if (n_keys > max_len) n_keys = max_len;
  if (n_keys < 0) n_keys = 0;
  const T* kbase = kc + ((long long)(b * Hkv + hk) * max_len) * DD + lane * 4;
  const T* vbase = vc + ((long long)(b * Hkv + hk) * max_len) * DD + lane * 4;
  float qv[4];
  {
    const T* qp = q + ((long long)b * H + h) * DD + lane * 4;
#pragma unroll
    for (int i = 0; i < 4; ++i) qv[i] = ToF<T>::to(qp[i]) * scale_log2;
  }
  float m = -INFINITY, l = 0.f, o[4] = {0.f, 0.f, 0.f, 0.f};
  // keys warp, warp + 8, ... in steps of 4 keys
  for (long long k0 = (long long)warp * 4; k0 < n_keys; k0 += kDecWarps * 4) {
    float s[4], vv[4][4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const long long key = k0 + u;
      float d = 0.f;
      if (key < n_keys) {
        const uint2 kr = *reinterpret_cast<const uint2*>(kbase + key * DD);
        const uint2 vr = *reinterpret_cast<const uint2*>(vbase + key * DD);
        const T* kp = reinterpret_cast<const T*>(&kr);
        const T* vp = reinterpret_cast<const T*>(&vr);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          d = fmaf(qv[i], ToF<T>::to(kp[i]), d);
          vv[u][i] = ToF<T>::to(vp[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) vv[u][i] = 0.f;
      }
      s[u] = d;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      s[u] = warp_sum(s[u]);
      if (k0 + u >= n_keys) s[u] = -INFINITY;
    }
    const float m_new = fmaxf(fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3])), m);
    const float alpha = exp2f(m - m_new);      // m_new is finite here: key k0 is always valid
    l *= alpha;
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] *= alpha;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float pz = exp2f(s[u] - m_new);
      l += pz;
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = fmaf(pz, vv[u][i], o[i]);
    }
    m = m_new;
  }
  if (lane == 0) { sh_m[warp] = m; sh_l[warp] = l; }
#pragma unroll
  for (int i = 0; i < 4; ++i) sh_o[warp][lane * 4 + i] = o[i];
  __syncthreads();
  if (threadIdx.x < DD) {
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) mm = fmaxf(mm, sh_m[w]);
    float ll = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float f = sh_m[w] == -INFINITY ? 0.f : exp2f(sh_m[w] - mm);
      ll += sh_l[w] * f;
      acc += sh_o[w][threadIdx.x] * f;
    }
    out[((long long)b * H + h) * DD + threadIdx.x] = ToF<T>::from(ll > 0.f ? acc / ll : 0.f);
  }
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int b200_decode_attention(int dtype, void* out, const void* q, const void* k_cache, const void* v_cache,
                                     const long long* pos, int B, int H, int Hkv, int max_len, int head_dim, float scale,
                                     cudaStream_t stream) {
  if (head_dim != DD || B <= 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0 || max_len <= 0) return (int)cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 7)
    return (int)cudaErrorNotSupported;
  const float sl2 = scale * 1.4426950408889634f;
  if (dtype == B200_BF16)
    decode_attn_kernel<__nv_bfloat16><<<B * H, kDecWarps * 32, 0, stream>>>((__nv_bfloat16*)out, (const __nv_bfloat16*)q,
        (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, pos, H, Hkv, max_len, sl2);
  else if (dtype == B200_F16)
    decode_attn_kernel<__half><<<B * H, kDecWarps * 32, 0, stream>>>((__half*)out, (const __half*)q, (const __half*)k_cache,
        (const __half*)v_cache, pos, H, Hkv, max_len, sl2);
  else
    return (int)cudaErrorNotSupported;
  B200K_LAUNCH_RET();
}
