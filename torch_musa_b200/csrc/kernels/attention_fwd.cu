// Flash-attention forward on the 5th-generation tensor cores (head_dim 128, bf16 / fp16, optional causal mask,
// grouped-query heads).
//
// One CTA owns 128 query rows of one (batch, head).  Per block of 128 keys:
//   S = Q K^T      tcgen05.mma M128 N128 K16 x 8, operands in 128B-swizzled shared memory (Q resident, K/V in a
//                  two-stage TMA ring), result in one of two 128-column TMEM buffers;
//   softmax        warps 2-5, one query row per thread: tcgen05.ld the row of S, scale into the log2 domain, causal /
//                  tail mask, running max and sum (no shuffles: the whole row is in one thread), P = exp2(S - max) is
//                  written as bf16 into shared memory in the swizzled K-major layout the tensor core expects;
//   O_blk = P V    tcgen05.mma with P as A operand and V (d contiguous) as MN-major B operand, fresh accumulation into
//                  a third TMEM buffer; the softmax threads add it to their fp32 output row in registers after
//                  rescaling by exp2(old max - new max).
// The MMA warp issues S for block j+1 before P V of block j, so the tensor core computes the next scores while
// the softmax warps work.  The epilogue divides by the row sum and writes O and the natural-log LSE.
// Every mbarrier wait is bounded (status word as for the GEMMs).
//
// Parity: the reference calls a closed vendor flash kernel (reference torch_musa/csrc/aten/ops/attention/mudnn/SDP.cpp:470-673).
#include "gemm_common.cuh"

#include <algorithm>

namespace b200k {
namespace {
using namespace gemmdev;

constexpr int AQ = 128, AK = 128, AD = 128;          // query rows, keys per block, head dim
constexpr int kTile = 128 * 128 * 2;                  // 32 KB: any of Q, K, V, P
constexpr int kAttnSmem = kTile /*Q*/ + 2 * 2 * kTile /*K,V x2*/ + kTile /*P*/ + 1024 + 256;
constexpr int kAttnThreads = 192;
constexpr uint32_t kAttnTmemCols = 512;               // S0, S1, O_blk (384 used)

struct AttnParams {
  int B, H, Hkv, Sq, Sk;
  int causal;
  float scale_log2;           // softmax scale * log2(e)
  int64_t o_sb, o_sh, o_ss;   // output strides in elements (last dim contiguous)
  float* lse;                 // [B, H, Sq]
  int q_blocks;
  int* status;
};

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, T* __restrict__ out, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;
  uint8_t* sK = smem + kTile;            // [2][kTile]
  uint8_t* sV = smem + 3 * kTile;        // [2][kTile]
  uint8_t* sP = smem + 5 * kTile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * kTile);
  uint64_t* q_full = bars;               // 1
  uint64_t* kv_full = bars + 1;          // [2]
  uint64_t* kv_empty = bars + 3;         // [2]
  uint64_t* s_full = bars + 5;           // [2]
  uint64_t* s_free = bars + 7;           // [2]  four softmax warps
  uint64_t* p_ready = bars + 9;          // four softmax warps
  uint64_t* p_free = bars + 10;          // tcgen05.commit
  uint64_t* o_full = bars + 11;          // tcgen05.commit
  uint64_t* o_free = bars + 12;          // four softmax warps
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late) query blocks first
  const int qb = p.q_blocks - 1 - (int)(blockIdx.x % p.q_blocks);
  const int bh = blockIdx.x / p.q_blocks;
  const int b = bh / p.H, h = bh - b * p.H;
  const int hk = h / (p.H / p.Hkv);
  const int q0 = qb * AQ;
  // keys this query block can see
  int k_end = p.Sk;
  if (p.causal) k_end = min(p.Sk, q0 + AQ);
  const int n_blocks = (k_end + AK - 1) / AK;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
      mbar_init(&s_full[s], 1);
      mbar_init(&s_free[s], 4);
    }
    mbar_init(p_ready, 4);
    mbar_init(p_free, 1);
    mbar_init(o_full, 1);
    mbar_init(o_free, 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kAttnTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, kTile);
      tma_load_4d(sQ, &tmap_q, q_full, 0, q0, h, b);            // d 0..63
      tma_load_4d(sQ + kTile / 2, &tmap_q, q_full, 64, q0, h, b);  // d 64..127
      for (int j = 0; j < n_blocks; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&kv_empty[st], (uint32_t)(((j >> 1) & 1) ^ 1), abort_flag)) break;
        mbar_expect_tx(&kv_full[st], 2 * kTile);
        const int k0 = j * AK;
        tma_load_4d(sK + st * kTile, &tmap_k, &kv_full[st], 0, k0, hk, b);
        tma_load_4d(sK + st * kTile + kTile / 2, &tmap_k, &kv_full[st], 64, k0, hk, b);
        // V as MN-major B operand: two boxes of 64 (d) x 128 (keys)
        tma_load_4d(sV + st * kTile, &tmap_v, &kv_full[st], 0, k0, hk, b);
        tma_load_4d(sV + st * kTile + kTile / 2, &tmap_v, &kv_full[st], 64, k0, hk, b);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptors: fp32 accumulate, bf16/fp16 operands, M128 N128; S: both K-major; PV: B MN-major
      const uint32_t fmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      const uint32_t idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_o = idesc_s | (1u << 16);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1, sb = j & 1;
        if (!mbar_wait(&kv_full[st], (uint32_t)((j >> 1) & 1), abort_flag)) return false;
        if (!mbar_wait(&s_free[sb], (uint32_t)(((j >> 1) & 1) ^ 1), abort_flag)) return false;
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + st * kTile);
#pragma unroll
        for (int kk = 0; kk < AD / 16; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * (kTile / 2) + (uint32_t)(kk & 3) * 32;   // 64-column atom, 32 B per k16
          umma_f16(tmem_base + (uint32_t)(sb * 128), make_desc(qa + off, 16, 1024), make_desc(ka + off, 16, 1024), idesc_s,
                   kk != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[sb]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, abort_flag) && n_blocks > 0 && issue_s(0);
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (j + 1 < n_blocks && !issue_s(j + 1)) { ok = false; break; }
        if (!mbar_wait(p_ready, (uint32_t)(j & 1), abort_flag)) { ok = false; break; }
        if (!mbar_wait(o_free, (uint32_t)((j & 1) ^ 1), abort_flag)) { ok = false; break; }
        tc_fence_after();
        const int st = j & 1;
        const uint32_t pa = smem_u32(sP), va = smem_u32(sV + st * kTile);
#pragma unroll
        for (int kk = 0; kk < AK / 16; ++kk) {
          // A = P (K-major over keys): two 64-key atoms; B = V (MN-major): 16 key rows = 2048 B, next 64-wide d box 16 KB on
          const uint32_t aoff = (uint32_t)(kk >> 2) * (kTile / 2) + (uint32_t)(kk & 3) * 32;
          umma_f16(tmem_o, make_desc(pa + aoff, 16, 1024), make_desc(va + (uint32_t)kk * 2048, kTile / 2, 1024), idesc_o,
                   kk != 0 ? 1u : 0u);
        }
        umma_commit(o_full);
        umma_commit(p_free);
        umma_commit(&kv_empty[st]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ softmax + output accumulation (warps 2..5)
    const int qw = warp & 3;
    const int r = qw * 32 + lane;            // query row inside the block = TMEM lane
    const int qi = q0 + r;
    float o[AD];
#pragma unroll
    for (int c = 0; c < AD; ++c) o[c] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks; ++j) {
      const int sb = j & 1;
      if (!mbar_wait(&s_full[sb], (uint32_t)((j >> 1) & 1), abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(qw * 32) << 16) + (uint32_t)(sb * 128);
      const int k0 = j * AK;
      // the row's visible keys: [0, lim)
      int lim = p.Sk - k0;
      if (p.causal) lim = min(lim, qi - k0 + 1);
      lim = max(0, min(lim, AK));
      // pass 1 over the row of S: the block maximum (the row is read from TMEM twice instead of being kept in
      // 128 registers next to the 128 output accumulators)
      float m_blk = -INFINITY;
#pragma unroll
      for (int c = 0; c < AK / 32; ++c) {
        uint32_t raw[32];
        tmem_ld32(taddr + (uint32_t)(c * 32), raw);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if (c * 32 + e < lim) m_blk = fmaxf(m_blk, __uint_as_float(raw[e]) * p.scale_log2);
      }
      const float m_new = fmaxf(m_run, m_blk);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;   // fully masked row so far
      const float alpha = exp2f(m_run - m_use);                // 0 when m_run = -inf
      float l_blk = 0.f;
      // P must not be overwritten while the previous P V still reads it
      if (!mbar_wait(p_free, (uint32_t)((j & 1) ^ 1), abort_flag)) { ok = false; break; }
      uint8_t* prow = sP + (size_t)r * 128;
      // pass 2: P = exp2(S - max) as bf16/fp16 into the swizzled K-major tile
#pragma unroll
      for (int c = 0; c < AK / 32; ++c) {
        uint32_t raw[32];
        tmem_ld32(taddr + (uint32_t)(c * 32), raw);
        tmem_ld_wait();
#pragma unroll
        for (int g8 = 0; g8 < 4; ++g8) {
          Vec16<T> pk;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int col = c * 32 + g8 * 8 + e;
            const float pv = col < lim ? exp2f(__uint_as_float(raw[g8 * 8 + e]) * p.scale_log2 - m_use) : 0.f;
            l_blk += pv;
            pk.v[e] = ToF<T>::from(pv);
          }
          const int c8 = c * 4 + g8;
          const int atom = c8 >> 3, ch = c8 & 7;
          *reinterpret_cast<Vec16<T>*>(prow + (size_t)atom * (kTile / 2) + (size_t)((ch ^ (r & 7)) * 16)) = pk;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[sb]);          // the tensor core may overwrite this S buffer
      l_run = l_run * alpha + l_blk;
      m_run = m_new;
      // make the generic-proxy writes of P visible to the tensor core (async proxy), then signal
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
      if (!mbar_wait(o_full, (uint32_t)(j & 1), abort_flag)) { ok = false; break; }
      tc_fence_after();
      const uint32_t oaddr = tmem_o + ((uint32_t)(qw * 32) << 16);
#pragma unroll
      for (int c = 0; c < AD / 32; ++c) {
        uint32_t raw[32];
        tmem_ld32(oaddr + (uint32_t)(c * 32), raw);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) o[c * 32 + e] = fmaf(o[c * 32 + e], alpha, __uint_as_float(raw[e]));
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free);
    }
    if (ok && qi < p.Sq) {
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      T* orow = out + (int64_t)b * p.o_sb + (int64_t)h * p.o_sh + (int64_t)qi * p.o_ss;
#pragma unroll
      for (int c8 = 0; c8 < AD / 8; ++c8) {
        Vec16<T> v;
#pragma unroll
        for (int e = 0; e < 8; ++e) v.v[e] = ToF<T>::from(o[c8 * 8 + e] * inv);
        st16(orow + c8 * 8, v);
      }
      if (p.lse) p.lse[((int64_t)b * p.H + h) * p.Sq + qi] = l_run > 0.f ? (m_run + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kAttnTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [B, H, S, D] view with element strides (sb, sh, ss, 1); box = 64 (d) x 128 (rows)
bool make_attn_map(CUtensorMap* out, const void* ptr, int bf16, int B, int H, int S, int64_t sb, int64_t sh, int64_t ss) {
  static EncodeTiledFn enc = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return (EncodeTiledFn) nullptr;
    }
    return (EncodeTiledFn)p;
  }();
  if (!enc) return false;
  cuuint64_t dims[4] = {(cuuint64_t)AD, (cuuint64_t)S, (cuuint64_t)H, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)ss * 2, (cuuint64_t)sh * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, 128, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(out, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, const_cast<void*>(ptr), dims,
             strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int b200_flash_attn_fwd(const b200_attn_t* a, void* out, float* lse, const void* q, const void* k,
                                   const void* v, cudaStream_t stream) {
  if (a->head_dim != AD || (a->dtype != B200_BF16 && a->dtype != B200_F16) || a->B <= 0 || a->H <= 0 || a->Hkv <= 0 ||
      a->H % a->Hkv != 0 || a->Sq <= 0 || a->Sk <= 0)
    return (int)cudaErrorNotSupported;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  auto st_ok = [](int64_t s) { return s % 8 == 0; };
  if (!al(q) || !al(k) || !al(v) || !al(out) || !st_ok(a->q_sb) || !st_ok(a->q_sh) || !st_ok(a->q_ss) || !st_ok(a->k_sb) ||
      !st_ok(a->k_sh) || !st_ok(a->k_ss) || !st_ok(a->v_sb) || !st_ok(a->v_sh) || !st_ok(a->v_ss) || !st_ok(a->o_sb) ||
      !st_ok(a->o_sh) || !st_ok(a->o_ss))
    return (int)cudaErrorNotSupported;
  // a broadcast (zero) stride cannot be a tensor-map stride
  if ((a->B > 1 && (a->q_sb == 0 || a->k_sb == 0 || a->v_sb == 0)) || (a->H > 1 && a->q_sh == 0) ||
      (a->Hkv > 1 && (a->k_sh == 0 || a->v_sh == 0)) || a->q_ss == 0 || a->k_ss == 0 || a->v_ss == 0)
    return (int)cudaErrorNotSupported;
  const int bf16 = a->dtype == B200_BF16;
  CUtensorMap mq, mk, mv;
  auto nz = [](int64_t s, int64_t fallback) { return s ? s : fallback; };
  if (!make_attn_map(&mq, q, bf16, a->B, a->H, a->Sq, nz(a->q_sb, 8), nz(a->q_sh, 8), a->q_ss) ||
      !make_attn_map(&mk, k, bf16, a->B, a->Hkv, a->Sk, nz(a->k_sb, 8), nz(a->k_sh, 8), a->k_ss) ||
      !make_attn_map(&mv, v, bf16, a->B, a->Hkv, a->Sk, nz(a->v_sb, 8), nz(a->v_sh, 8), a->v_ss))
    return (int)cudaErrorNotSupported;
  AttnParams p{};
  p.B = a->B; p.H = a->H; p.Hkv = a->Hkv; p.Sq = a->Sq; p.Sk = a->Sk;
  p.causal = a->causal;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.o_sb = a->o_sb; p.o_sh = a->o_sh; p.o_ss = a->o_ss;
  p.lse = lse;
  p.q_blocks = (a->Sq + AQ - 1) / AQ;
  p.status = gemm_status_word_device();
  const long long grid = (long long)a->B * a->H * p.q_blocks;
  if (grid > 2147483647ll) return (int)cudaErrorNotSupported;
  if (bf16) {
    static bool set = false;
    auto kern = attn_fwd_kernel<__nv_bfloat16>;
    if (!set) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem);
      if (e != cudaSuccess) return (int)e;
      set = true;
    }
    kern<<<(unsigned)grid, kAttnThreads, kAttnSmem, stream>>>(mq, mk, mv, (__nv_bfloat16*)out, p);
  } else {
    static bool set = false;
    auto kern = attn_fwd_kernel<__half>;
    if (!set) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnSmem);
      if (e != cudaSuccess) return (int)e;
      set = true;
    }
    kern<<<(unsigned)grid, kAttnThreads, kAttnSmem, stream>>>(mq, mk, mv, (__half*)out, p);
  }
  B200K_LAUNCH_RET();
}
