// Single-query ("decode") attention over a static KV cache, head_dim 128.
//
// One CTA per (batch, query head), eight warps.  A warp is four independent groups of eight lanes; a group owns
// every 32nd key of [0, *pos] and its lanes split the 128 dimensions sixteen each (two 16-byte loads per row), so
// a score needs three shuffles instead of a full warp reduction and the probability never has to be broadcast:
// every group runs its own online softmax (log2 domain) and accumulates its own output slice.  Two keys per group
// are in flight per iteration.  The 32 partial (max, sum, output) triples of a CTA are merged through shared memory.
// The visible length is read from device memory, so the kernel can sit inside a captured graph and follow the
// position counter without any host involvement.  Memory-bound by design: K and V are read exactly once per query
// head (grouped-query heads re-read their shared KV head through L2).
// Parity: the reference has no decode kernel; it relies on the vendor SDPA (reference
// torch_musa/csrc/aten/ops/attention/mudnn/SDP.cpp).
#include "common.cuh"

namespace b200k {
namespace {

constexpr int DD = 128;
constexpr int kDecWarps = 8;
constexpr int kGroups = 4;              // lane groups per warp
constexpr int kDimsPerLane = 16;        // 128 dims / 8 lanes
constexpr int kParts = kDecWarps * kGroups;

template <typename T>
__device__ __forceinline__ void load16(const T* p, float (&out)[kDimsPerLane]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint4 b = *reinterpret_cast<const uint4*>(p + 8);
  const T* pa = reinterpret_cast<const T*>(&a);
  const T* pb = reinterpret_cast<const T*>(&b);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    out[i] = ToF<T>::to(pa[i]);
    out[8 + i] = ToF<T>::to(pb[i]);
  }
}

// One lane's sixteen elements of a cache row, kept packed (two 16-byte words) until use.
template <typename T>
struct Row {
  uint4 a, b;
  __device__ __forceinline__ void load(const T* p, bool valid) {
    if (valid) {
      a = *reinterpret_cast<const uint4*>(p);
      b = *reinterpret_cast<const uint4*>(p + 8);
    } else {
      a = make_uint4(0, 0, 0, 0);
      b = a;
    }
  }
  __device__ __forceinline__ float get(int i) const {
    const T* pa = reinterpret_cast<const T*>(&a);
    const T* pb = reinterpret_cast<const T*>(&b);
    return ToF<T>::to(i < 8 ? pa[i] : pb[i - 8]);
  }
};

template <typename T>
__global__ void __launch_bounds__(kDecWarps * 32, 2)
decode_attn_kernel(T* __restrict__ out, const T* __restrict__ q, const T* __restrict__ kc, const T* __restrict__ vc,
                   const long long* __restrict__ pos_ptr, int H, int Hkv, int max_len, float scale_log2) {
  __shared__ float sh_m[kParts], sh_l[kParts];
  __shared__ float sh_o[kParts][DD];
  const int b = blockIdx.x / H, h = blockIdx.x - b * H;
  const int hk = h / (H / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane >> 3, gl = lane & 7;
  const int part = warp * kGroups + grp;
  long long n_keys = *pos_ptr + 1;
  if (n_keys > max_len) n_keys = max_len;
  if (n_keys < 0) n_keys = 0;
  const T* kbase = kc + ((long long)(b * Hkv + hk) * max_len) * DD + gl * kDimsPerLane;
  const T* vbase = vc + ((long long)(b * Hkv + hk) * max_len) * DD + gl * kDimsPerLane;
  float qv[kDimsPerLane];
  load16(q + ((long long)b * H + h) * DD + gl * kDimsPerLane, qv);
#pragma unroll
  for (int i = 0; i < kDimsPerLane; ++i) qv[i] *= scale_log2;
  float m = -INFINITY, l = 0.f, o[kDimsPerLane];
#pragma unroll
  for (int i = 0; i < kDimsPerLane; ++i) o[i] = 0.f;

  auto consume = [&](const Row<T>& kr, const Row<T>& vr, bool valid) {
    float d = 0.f;
#pragma unroll
    for (int i = 0; i < kDimsPerLane; ++i) d = fmaf(qv[i], kr.get(i), d);
    d += __shfl_xor_sync(0xffffffffu, d, 4);
    d += __shfl_xor_sync(0xffffffffu, d, 2);
    d += __shfl_xor_sync(0xffffffffu, d, 1);
    if (!valid) return;
    const float m_new = fmaxf(m, d);
    const float alpha = exp2f(m - m_new);    // m = -inf on the first key: alpha = 0, the empty state vanishes
    const float pz = exp2f(d - m_new);
    l = fmaf(l, alpha, pz);
#pragma unroll
    for (int i = 0; i < kDimsPerLane; ++i) o[i] = fmaf(pz, vr.get(i), o[i] * alpha);
    m = m_new;
  };

  // keys part, part + 32, ...; two in flight, kept packed until they are consumed.  The shuffles inside `consume`
  // are executed by every lane of the warp: a group without a key left feeds zeros through them and skips the update.
  const long long span = 2 * kParts;
  const long long k_end = ((n_keys + span - 1) / span) * span;
  for (long long k0 = part; k0 < k_end; k0 += span) {
    const long long ka = k0, kb = k0 + kParts;
    const bool va = ka < n_keys, vb = kb < n_keys;
    Row<T> k_a, v_a, k_b, v_b;
    k_a.load(kbase + ka * DD, va);
    v_a.load(vbase + ka * DD, va);
    k_b.load(kbase + kb * DD, vb);
    v_b.load(vbase + kb * DD, vb);
    consume(k_a, v_a, va);
    consume(k_b, v_b, vb);
  }
  if (gl == 0) { sh_m[part] = m; sh_l[part] = l; }
#pragma unroll
  for (int i = 0; i < kDimsPerLane; ++i) sh_o[part][gl * kDimsPerLane + i] = o[i];
  __syncthreads();
  if (threadIdx.x < DD) {
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kParts; ++w) mm = fmaxf(mm, sh_m[w]);
    float ll = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < kParts; ++w) {
      const float f = sh_m[w] == -INFINITY ? 0.f : exp2f(sh_m[w] - mm);
      ll += sh_l[w] * f;
      acc += sh_o[w][threadIdx.x] * f;
    }
    out[((long long)b * H + h) * DD + threadIdx.x] = ToF<T>::from(ll > 0.f ? acc / ll : 0.f);
  }
}

// One decode step's rotary embedding and cache update in ONE launch: the new query rows are rotated into q_out, the
// new key rows are rotated straight into the key cache at position *pos, the new value rows are copied into the value
// cache.  One warp per (batch, head) row of 128 elements: a lane owns two adjacent dims of the first half and their
// partners in the second half (rotate-half layout).  The position is read from device memory (graph-capturable).
template <typename T>
__global__ void __launch_bounds__(256)
decode_rope_cache_kernel(T* __restrict__ q_out, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                         long long q_sb, long long q_sh, long long k_sb, long long k_sh, long long v_sb, long long v_sh,
                         const float* __restrict__ cosv, const float* __restrict__ sinv, const long long* __restrict__ pos_ptr,
                         T* __restrict__ k_cache, T* __restrict__ v_cache, int B, int H, int Hkv, int max_len, int table_len) {
  const int per_b = H + 2 * Hkv;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= (long long)B * per_b) return;
  const int lane = threadIdx.x & 31;
  const int b = (int)(row / per_b), j = (int)(row - (long long)b * per_b);
  long long p = *pos_ptr;
  p = p < 0 ? 0 : (p >= max_len ? max_len - 1 : p);
  const long long pt = p < table_len ? p : table_len - 1;
  const T* src;
  T* dst;
  bool rotate = true;
  if (j < H) {
    src = q + b * q_sb + j * q_sh;
    dst = q_out + ((long long)b * H + j) * DD;
  } else if (j < H + Hkv) {
    const int hk = j - H;
    src = k + b * k_sb + hk * k_sh;
    dst = k_cache + (((long long)b * Hkv + hk) * max_len + p) * DD;
  } else {
    const int hk = j - H - Hkv;
    src = v + b * v_sb + hk * v_sh;
    dst = v_cache + (((long long)b * Hkv + hk) * max_len + p) * DD;
    rotate = false;
  }
  // two adjacent elements (4 bytes) of each half
  const uint32_t lo = *reinterpret_cast<const uint32_t*>(src + lane * 2);
  const uint32_t hi = *reinterpret_cast<const uint32_t*>(src + DD / 2 + lane * 2);
  if (!rotate) {
    *reinterpret_cast<uint32_t*>(dst + lane * 2) = lo;
    *reinterpret_cast<uint32_t*>(dst + DD / 2 + lane * 2) = hi;
    return;
  }
  const T* l2 = reinterpret_cast<const T*>(&lo);
  const T* h2 = reinterpret_cast<const T*>(&hi);
  const float2 c = *reinterpret_cast<const float2*>(cosv + pt * (DD / 2) + lane * 2);
  const float2 sn = *reinterpret_cast<const float2*>(sinv + pt * (DD / 2) + lane * 2);
  const float x0a = ToF<T>::to(l2[0]), x0b = ToF<T>::to(l2[1]), x1a = ToF<T>::to(h2[0]), x1b = ToF<T>::to(h2[1]);
  T ol[2], oh[2];
  ol[0] = ToF<T>::from(x0a * c.x - x1a * sn.x);
  ol[1] = ToF<T>::from(x0b * c.y - x1b * sn.y);
  oh[0] = ToF<T>::from(x1a * c.x + x0a * sn.x);
  oh[1] = ToF<T>::from(x1b * c.y + x0b * sn.y);
  *reinterpret_cast<uint32_t*>(dst + lane * 2) = *reinterpret_cast<const uint32_t*>(ol);
  *reinterpret_cast<uint32_t*>(dst + DD / 2 + lane * 2) = *reinterpret_cast<const uint32_t*>(oh);
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int b200_decode_attention(int dtype, void* out, const void* q, const void* k_cache, const void* v_cache,
                                     const long long* pos, int B, int H, int Hkv, int max_len, int head_dim, float scale,
                                     cudaStream_t stream) {
  if (head_dim != DD || B <= 0 || H <= 0 || Hkv <= 0 || H % Hkv != 0 || max_len <= 0) return (int)cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15)
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

extern "C" int b200_decode_rope_cache(int dtype, void* q_out, const void* q, const void* k, const void* v, const int64_t* strides,
                                      const float* cosv, const float* sinv, const long long* pos, void* k_cache, void* v_cache,
                                      int B, int H, int Hkv, int max_len, int head_dim, int table_len, cudaStream_t stream) {
  // strides (elements): q batch, q head, k batch, k head, v batch, v head; rows of 128 contiguous elements, 4-byte aligned
  if (head_dim != DD || B <= 0 || H <= 0 || Hkv <= 0 || max_len <= 0 || table_len <= 0) return (int)cudaErrorNotSupported;
  for (int i = 0; i < 6; ++i)
    if (strides[i] % 2 != 0) return (int)cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 3)
    return (int)cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(cosv) | reinterpret_cast<uintptr_t>(sinv)) & 7) return (int)cudaErrorNotSupported;
  const long long rows = (long long)B * (H + 2 * Hkv);
  const unsigned grid = (unsigned)((rows + 7) / 8);
  if (dtype == B200_BF16)
    decode_rope_cache_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(
        (__nv_bfloat16*)q_out, (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, strides[0], strides[1],
        strides[2], strides[3], strides[4], strides[5], cosv, sinv, pos, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, B, H,
        Hkv, max_len, table_len);
  else if (dtype == B200_F16)
    decode_rope_cache_kernel<__half><<<grid, 256, 0, stream>>>(
        (__half*)q_out, (const __half*)q, (const __half*)k, (const __half*)v, strides[0], strides[1], strides[2], strides[3],
        strides[4], strides[5], cosv, sinv, pos, (__half*)k_cache, (__half*)v_cache, B, H, Hkv, max_len, table_len);
  else
    return (int)cudaErrorNotSupported;
  B200K_LAUNCH_RET();
}
