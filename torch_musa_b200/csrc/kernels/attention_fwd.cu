// Flash-attention forward on the 5th-generation tensor cores (head_dim 128, bf16 / fp16, optional causal mask,
// grouped-query heads): two query tiles per CTA in ping-pong, scores and the output accumulators in TMEM, K / V through
// a TMA ring, every mbarrier wait bounded (status word as for the GEMMs).  The kernel comment below has the pipeline.
//
// Parity: the reference calls a closed vendor flash kernel (reference torch_musa/csrc/aten/ops/attention/mudnn/SDP.cpp:470-673).
#include "attention_common.cuh"

#include <algorithm>

namespace b200k {
namespace {
using namespace gemmdev;
using namespace attndev;

constexpr int AQ = 128, AK = 128, AD = 128;          // query rows per tile, keys per block, head dim
constexpr int kTile = 128 * 128 * 2;                  // 32 KB: any of Q, K, V, P
constexpr int kRing = 3;                              // K / V tiles in flight
constexpr int kAttnSmem = 2 * kTile /*Q0,Q1*/ + kRing * kTile + 2 * kTile /*P0,P1*/ + 1024 + 256;
constexpr int kAttnThreads = 320;                     // 2 softmax warpgroups, TMA warp, MMA warp
constexpr uint32_t kAttnTmemCols = 512;               // S0, S1, O0, O1
constexpr float kRescaleThreshold = 8.f;              // log2 domain: P stays below 2^8

struct AttnParams {
  int B, H, Hkv, Sq, Sk;
  int causal;
  float scale_log2;           // softmax scale * log2(e)
  int64_t o_sb, o_sh, o_ss;   // output strides in elements (last dim contiguous)
  float* lse;                 // [B, H, Sq]; packed sequences: [H, total_q]
  int q_blocks, q_pairs;
  // packed variable-length sequences (NULL: dense batch): sequence b holds rows [cu_q[b], cu_q[b + 1]) of the packed
  // q / out [total_q, H, 128] and rows [cu_k[b], cu_k[b + 1]) of k / v; Sq / Sk are then the longest lengths
  const int* cu_q;
  const int* cu_k;
  int total_q;
  int* status;
};

// One CTA owns two adjacent 128-row query tiles of one (batch, head).  Per block of 128 keys and per tile t:
//   S_t = Q_t K^T     tcgen05.mma M128 N128 K16 x 8 into TMEM (operands in 128B-swizzled shared memory);
//   softmax           warpgroup t, one query row per thread: two passes over the row of S in TMEM (block maximum, then
//                     P = exp2(S * scale - m) as bf16 into shared memory in the layout of an A operand);
//   O_t += P_t V      tcgen05.mma accumulating in TMEM over all key blocks.
// The exponent's reference maximum m is only raised when the running maximum has grown by more than 2^8 ("lazy"
// rescaling): then the warpgroup multiplies its rows of O in TMEM (tcgen05.ld / st) before it releases P.  That is rare
// after the first blocks, so O normally never leaves TMEM until the epilogue.
// The MMA warp alternates between the tiles (P V of tile 0, next S of tile 0, P V of tile 1, next S of tile 1), so one
// tile's softmax runs while the tensor core works for the other; K and V tiles stream through a three-slot TMA ring.
template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, T* __restrict__ out, const AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sQ = smem;                          // [2][kTile]
  uint8_t* sR = smem + 2 * kTile;              // [kRing][kTile]
  uint8_t* sP = smem + (2 + kRing) * kTile;    // [2][kTile]
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (4 + kRing) * kTile);
  uint64_t* q_full = bars;                     // [2]
  uint64_t* r_full = bars + 2;                 // [kRing]
  uint64_t* r_empty = bars + 2 + kRing;        // [kRing]  tcgen05.commit
  uint64_t* s_full = bars + 2 + 2 * kRing;     // [2]      tcgen05.commit
  uint64_t* s_free = s_full + 2;               // [2]      four softmax warps
  uint64_t* p_ready = s_free + 2;              // [2]      four softmax warps
  uint64_t* pv_done = p_ready + 2;             // [2]      tcgen05.commit
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // heavy (late) query tiles first, across all (batch, head) instances
  const int n_bh = p.B * p.H;
  const int qp = p.q_pairs - 1 - (int)(blockIdx.x / n_bh);
  const int bh = (int)(blockIdx.x % n_bh);
  const int b = bh / p.H, h = bh - b * p.H;
  const int hk = h / (p.H / p.Hkv);
  // this instance's sequence: lengths, first packed rows and the batch coordinate of the tensor maps.  Rows past a
  // packed sequence's end belong to the next sequence: they are loaded, masked by index and never stored.
  int Sq = p.Sq, Sk = p.Sk, qoff = 0, koff = 0, bt = b;
  if (p.cu_q) {
    qoff = p.cu_q[b];
    Sq = p.cu_q[b + 1] - qoff;
    koff = p.cu_k[b];
    Sk = p.cu_k[b + 1] - koff;
    bt = 0;
  }
  int nb[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int q0 = (2 * qp + t) * AQ;
    int k_end = Sk;
    if (p.causal) k_end = min(Sk, q0 + AQ);
    nb[t] = q0 < Sq ? (k_end + AK - 1) / AK : 0;
  }
  const int nbmax = max(nb[0], nb[1]);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int t = 0; t < 2; ++t) {
      mbar_init(&q_full[t], 1);
      mbar_init(&s_full[t], 1);
      mbar_init(&s_free[t], 4);
      mbar_init(&p_ready[t], 4);
      mbar_init(&pv_done[t], 1);
    }
    for (int s = 0; s < kRing; ++s) {
      mbar_init(&r_full[s], 1);
      mbar_init(&r_empty[s], 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, kAttnTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int t = 0; t < 2; ++t) {
        if (nb[t] == 0) continue;
        const int q0 = (2 * qp + t) * AQ;
        mbar_expect_tx(&q_full[t], kTile);
        tma_load_4d(sQ + t * kTile, &tmap_q, &q_full[t], 0, qoff + q0, h, bt);                 // d 0..63
        tma_load_4d(sQ + t * kTile + kTile / 2, &tmap_q, &q_full[t], 64, qoff + q0, h, bt);    // d 64..127
      }
      for (int n = 0; n < 2 * nbmax; ++n) {
        const int st = n % kRing;
        if (!mbar_wait(&r_empty[st], (uint32_t)(((n / kRing) & 1) ^ 1), abort_flag)) break;
        mbar_expect_tx(&r_full[st], kTile);
        const int k0 = (n >> 1) * AK;
        const CUtensorMap* map = (n & 1) ? &tmap_v : &tmap_k;   // V is read as an MN-major B operand: same boxes
        tma_load_4d(sR + st * kTile, map, &r_full[st], 0, koff + k0, hk, bt);
        tma_load_4d(sR + st * kTile + kTile / 2, map, &r_full[st], 64, koff + k0, hk, bt);
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // instruction descriptors: fp32 accumulate, bf16/fp16 operands, M128 N128; S: both K-major; PV: B MN-major
      const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      const uint32_t idesc_s = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_o = idesc_s | (1u << 16);
      bool ok = true;
      auto ring_wait = [&](int n) { return mbar_wait(&r_full[n % kRing], (uint32_t)((n / kRing) & 1), abort_flag); };
      auto issue_s = [&](int t, int n) {     // S_t = Q_t K^T with K in ring item n
        const uint32_t qa = smem_u32(sQ + t * kTile), ka = smem_u32(sR + (n % kRing) * kTile);
#pragma unroll
        for (int kk = 0; kk < AD / 16; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * (kTile / 2) + (uint32_t)(kk & 3) * 32;   // 64-column atom, 32 B per k16
          umma_f16(tmem_base + (uint32_t)(t * 128), make_desc(qa + off, 16, 1024), make_desc(ka + off, 16, 1024), idesc_s,
                   kk != 0 ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
      };
      auto issue_pv = [&](int t, int n, bool first) {   // O_t (+)= P_t V with V in ring item n
        const uint32_t pa = smem_u32(sP + t * kTile), va = smem_u32(sR + (n % kRing) * kTile);
#pragma unroll
        for (int kk = 0; kk < AK / 16; ++kk) {
          // A = P (K-major over keys): two 64-key atoms; B = V (MN-major): 16 key rows = 2048 B, next 64-wide d box 16 KB on
          const uint32_t aoff = (uint32_t)(kk >> 2) * (kTile / 2) + (uint32_t)(kk & 3) * 32;
          umma_f16(tmem_base + 256u + (uint32_t)(t * 128), make_desc(pa + aoff, 16, 1024),
                   make_desc(va + (uint32_t)kk * 2048, kTile / 2, 1024), idesc_o, (first && kk == 0) ? 0u : 1u);
        }
        umma_commit(&pv_done[t]);
      };
      for (int t = 0; t < 2 && ok; ++t)
        if (nb[t] > 0) ok = mbar_wait(&q_full[t], 0, abort_flag);
      if (ok && nbmax > 0) ok = ring_wait(0);
      if (ok && nbmax > 0) {
        tc_fence_after();
        for (int t = 0; t < 2; ++t)
          if (nb[t] > 0) issue_s(t, 0);
        umma_commit(&r_empty[0]);
      }
      for (int j = 0; j < nbmax && ok; ++j) {
        const int nv = 2 * j + 1, nk = 2 * j + 2;
        if (!ring_wait(nv)) { ok = false; break; }
        bool k_ready = false;
        for (int t = 0; t < 2 && ok; ++t) {
          if (j < nb[t]) {
            if (!mbar_wait(&p_ready[t], (uint32_t)(j & 1), abort_flag)) { ok = false; break; }
            tc_fence_after();
            issue_pv(t, nv, j == 0);
          }
          if (j + 1 < nb[t]) {
            if (!k_ready) {
              if (!ring_wait(nk)) { ok = false; break; }
              k_ready = true;
            }
            if (!mbar_wait(&s_free[t], (uint32_t)(j & 1), abort_flag)) { ok = false; break; }
            tc_fence_after();
            issue_s(t, nk);
          }
        }
        if (!ok) break;
        umma_commit(&r_empty[nv % kRing]);
        if (j + 1 < nbmax) umma_commit(&r_empty[nk % kRing]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ softmax warpgroup t (warps 4t .. 4t+3)
    const int t = warp >> 2;
    const int qw = warp & 3;                 // TMEM lane quarter of this warp
    const int r = qw * 32 + lane;            // query row inside the tile = TMEM lane
    const int qi = (2 * qp + t) * AQ + r;
    const uint32_t lane_base = ((uint32_t)(qw * 32) << 16);
    const uint32_t s_addr = tmem_base + lane_base + (uint32_t)(t * 128);
    const uint32_t o_addr = tmem_base + lane_base + 256u + (uint32_t)(t * 128);
    uint8_t* prow = sP + t * kTile + (size_t)r * 128;
    float m_ref = -INFINITY;                 // maximum the exponents refer to (raised lazily)
    float l_run = 0.f;
    bool ok = true;
    const int n_blocks = nb[t];
    // warp-uniform wait: the warp-collective TMEM accesses and votes below need all 32 lanes to take the same path
    auto wait_all = [&](uint64_t* bar, uint32_t parity) {
      const bool w = mbar_wait(bar, parity, abort_flag);
      return __all_sync(0xffffffffu, w);
    };
    for (int j = 0; j < n_blocks; ++j) {
      if (!wait_all(&s_full[t], (uint32_t)(j & 1))) { ok = false; break; }
      tc_fence_after();
      const int k0 = j * AK;
      // the row's visible keys: [0, lim)
      int lim = Sk - k0;
      if (p.causal) lim = min(lim, qi - k0 + 1);
      lim = max(0, min(lim, AK));
      const bool full = __all_sync(0xffffffffu, lim == AK);
      // pass 1: block maximum of the raw scores (the TMEM load of one 32-column chunk overlaps the work on the other)
      float m_blk = -INFINITY;
      {
        uint32_t ra[32], rb[32];
        auto chunk_max = [&](const uint32_t (&raw)[32], int c) {
          if (full) {
#pragma unroll
            for (int e = 0; e < 32; ++e) m_blk = fmaxf(m_blk, __uint_as_float(raw[e]));
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (c * 32 + e < lim) m_blk = fmaxf(m_blk, __uint_as_float(raw[e]));
          }
        };
        tmem_ld32(s_addr, ra);
        tmem_ld_wait();
        tmem_ld32(s_addr + 32u, rb);
        chunk_max(ra, 0);
        tmem_ld_wait();
        tmem_ld32(s_addr + 64u, ra);
        chunk_max(rb, 1);
        tmem_ld_wait();
        tmem_ld32(s_addr + 96u, rb);
        chunk_max(ra, 2);
        tmem_ld_wait();
        chunk_max(rb, 3);
      }
      const float m_new = fmaxf(m_ref, m_blk * p.scale_log2);
      // P of the previous block must have been consumed (and O updated) before P is rewritten or O rescaled
      if (j > 0 && !wait_all(&pv_done[t], (uint32_t)((j - 1) & 1))) { ok = false; break; }
      const bool raise = m_new - m_ref > kRescaleThreshold;      // also true for the first finite maximum
      if (__any_sync(0xffffffffu, raise)) {
        const float alpha = raise ? exp2f(m_ref - m_new) : 1.f;   // 0 when m_ref = -inf
        if (j > 0) {
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < AD / 32; ++c) {
            uint32_t raw[32];
            tmem_ld32(o_addr + (uint32_t)(c * 32), raw);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) raw[e] = __float_as_uint(__uint_as_float(raw[e]) * alpha);
            tmem_st32(o_addr + (uint32_t)(c * 32), raw);
          }
          tmem_st_wait();
        }
        if (raise) {
          l_run *= alpha;
          m_ref = m_new;
        }
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;       // row without any visible key so far
      // pass 2: P = exp2(S * scale - m) as bf16/fp16 into the swizzled K-major tile; packed fp32 arithmetic, one
      // special-function instruction per exponential, one conversion per pair
      float l0 = 0.f, l1 = 0.f;
      {
        uint32_t ra[32], rb[32];
        const float neg_m = -m_use;
        auto chunk_p = [&](const uint32_t (&raw)[32], int c) {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            float x0, x1;
            fma2(x0, x1, __uint_as_float(raw[e]), __uint_as_float(raw[e + 1]), p.scale_log2, neg_m);
            float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
            if (!full) {
              if (c * 32 + e >= lim) p0 = 0.f;
              if (c * 32 + e + 1 >= lim) p1 = 0.f;
            }
            add2(l0, l1, p0, p1);
            pk[e >> 1] = pack2<T>(p0, p1);
          }
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            const int c8 = c * 4 + g8;
            const int atom = c8 >> 3, ch = c8 & 7;
            *reinterpret_cast<uint4*>(prow + (size_t)atom * (kTile / 2) + (size_t)((ch ^ (r & 7)) * 16)) =
                make_uint4(pk[g8 * 4], pk[g8 * 4 + 1], pk[g8 * 4 + 2], pk[g8 * 4 + 3]);
          }
        };
        tmem_ld32(s_addr, ra);
        tmem_ld_wait();
        tmem_ld32(s_addr + 32u, rb);
        chunk_p(ra, 0);
        tmem_ld_wait();
        tmem_ld32(s_addr + 64u, ra);
        chunk_p(rb, 1);
        tmem_ld_wait();
        tmem_ld32(s_addr + 96u, rb);
        chunk_p(ra, 2);
        tmem_ld_wait();
        chunk_p(rb, 3);
      }
      const float l_blk = l0 + l1;
      l_run += l_blk;
      tc_fence_before();
      // make the generic-proxy writes of P visible to the tensor core (async proxy), then signal
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_free[t]);          // the tensor core may overwrite this S buffer
        mbar_arrive(&p_ready[t]);
      }
    }
    if (ok && n_blocks > 0) ok = wait_all(&pv_done[t], (uint32_t)((n_blocks - 1) & 1));
    if (ok && n_blocks > 0) {
      tc_fence_after();
      const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
      T* orow = out + (int64_t)bt * p.o_sb + (int64_t)h * p.o_sh + (int64_t)(qoff + qi) * p.o_ss;
#pragma unroll
      for (int c = 0; c < AD / 32; ++c) {
        uint32_t raw[32];
        tmem_ld32(o_addr + (uint32_t)(c * 32), raw);
        tmem_ld_wait();
        if (qi < Sq) {
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            Vec16<T> v;
#pragma unroll
            for (int e = 0; e < 8; ++e) v.v[e] = ToF<T>::from(__uint_as_float(raw[g8 * 8 + e]) * inv);
            st16(orow + c * 32 + g8 * 8, v);
          }
        }
      }
      if (qi < Sq && p.lse)
        p.lse[p.cu_q ? (int64_t)h * p.total_q + qoff + qi : ((int64_t)b * p.H + h) * p.Sq + qi] = l_run > 0.f ? (m_ref + log2f(l_run)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kAttnTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
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
  if ((a->B > 1 && !a->cu_seqlens_q && (a->q_sb == 0 || a->k_sb == 0 || a->v_sb == 0)) || (a->H > 1 && a->q_sh == 0) ||
      (a->Hkv > 1 && (a->k_sh == 0 || a->v_sh == 0)) || a->q_ss == 0 || a->k_ss == 0 || a->v_ss == 0)
    return (int)cudaErrorNotSupported;
  const int bf16 = a->dtype == B200_BF16;
  CUtensorMap mq, mk, mv;
  auto nz = [](int64_t s, int64_t fallback) { return s ? s : fallback; };
  const bool packed = a->cu_seqlens_q != nullptr;
  if (packed) {
    if (!a->cu_seqlens_k || a->total_q <= 0 || a->total_k <= 0) return (int)cudaErrorNotSupported;
    // one "batch" of total rows: the kernel adds each sequence's first row to its tile coordinates
    if (!make_attn_map(&mq, q, bf16, 1, a->H, a->total_q, (int64_t)a->total_q * a->q_ss, nz(a->q_sh, 8), a->q_ss) ||
        !make_attn_map(&mk, k, bf16, 1, a->Hkv, a->total_k, (int64_t)a->total_k * a->k_ss, nz(a->k_sh, 8), a->k_ss) ||
        !make_attn_map(&mv, v, bf16, 1, a->Hkv, a->total_k, (int64_t)a->total_k * a->v_ss, nz(a->v_sh, 8), a->v_ss))
      return (int)cudaErrorNotSupported;
  } else if (!make_attn_map(&mq, q, bf16, a->B, a->H, a->Sq, nz(a->q_sb, 8), nz(a->q_sh, 8), a->q_ss) ||
             !make_attn_map(&mk, k, bf16, a->B, a->Hkv, a->Sk, nz(a->k_sb, 8), nz(a->k_sh, 8), a->k_ss) ||
             !make_attn_map(&mv, v, bf16, a->B, a->Hkv, a->Sk, nz(a->v_sb, 8), nz(a->v_sh, 8), a->v_ss))
    return (int)cudaErrorNotSupported;
  AttnParams p{};
  p.B = a->B; p.H = a->H; p.Hkv = a->Hkv; p.Sq = a->Sq; p.Sk = a->Sk;
  p.causal = a->causal;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.o_sb = a->o_sb; p.o_sh = a->o_sh; p.o_ss = a->o_ss;
  p.lse = lse;
  p.cu_q = a->cu_seqlens_q;
  p.cu_k = a->cu_seqlens_k;
  p.total_q = a->total_q;
  p.q_blocks = (a->Sq + AQ - 1) / AQ;
  p.q_pairs = (p.q_blocks + 1) / 2;
  p.status = gemm_status_word_device();
  const long long grid = (long long)a->B * a->H * p.q_pairs;
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
