// Flash-attention backward on the 5th-generation tensor cores (head_dim 128, bf16 / fp16, optional causal mask,
// grouped-query heads).
//
// One CTA owns one block of 128 keys of one (batch, kv head); K and V stay resident in shared memory, dK and dV
// accumulate in TMEM over every query block (and every query head of the group) that sees the keys.  Everything is
// computed transposed, keys along the 128 TMEM lanes, so that one thread owns one key row:
//   S^T  = K Q^T          tcgen05.mma, both operands K-major                         -> TMEM columns [0, 128)
//   dP^T = V dO^T         the same shape                                             -> TMEM columns [128, 256)
//   P^T  = exp2(S^T * scale - lse[q]),  dS^T = P^T * (dP^T - delta[q]) * scale       two warpgroups, half of the
//                         query columns each; both written as bf16 into shared memory in the layout of an A operand
//   dV  += P^T dO         A = P^T (K-major over queries), B = dO read MN-major       -> TMEM columns [256, 384)
//   dK  += dS^T Q         A = dS^T, B = Q read MN-major                              -> TMEM columns [384, 512)
//   dQ   = dS K           A = dS^T read MN-major, B = K read MN-major, fresh         -> TMEM columns [128, 256) again
// dQ of this (query block, key block) pair is staged as fp32 in the shared memory that P^T / dS^T occupied and added
// to an fp32 buffer in global memory by TMA reductions (cp.reduce.async.bulk.tensor ... add); the caller zeroes that
// buffer and converts it afterwards.  delta = rowsum(dO * O) comes
// from a small preprocessing kernel.  Q and dO stream through a three-slot TMA ring; every wait is bounded.
//
// Parity: the reference calls a closed vendor flash backward (reference torch_musa/csrc/aten/ops/attention/mudnn/SDP.cpp:678-845).
#include "attention_common.cuh"

#include <algorithm>

namespace b200k {
namespace {
using namespace gemmdev;
using namespace attndev;

constexpr int BQ = 128, BK = 128, BD = 128;
constexpr int kTile = 128 * 128 * 2;
constexpr int kRing = 3;
constexpr int kBwdSmem = 2 * kTile /*K, V*/ + kRing * kTile /*Q, dO ring*/ + 2 * kTile /*P^T, dS^T*/ + 1024 +
                         2 * 128 * 4 /*lse, delta*/ + 128;
static_assert(kBwdSmem <= 232448, "exceeds the 227 KB of shared memory a CTA can have");
constexpr int kBwdThreads = 320;
constexpr uint32_t kBwdTmemCols = 512;

struct BwdParams {
  int B, H, Hkv, Sq, Sk;
  int causal;
  float scale, scale_log2;
  const float* lse;       // [B, H, Sq] natural log
  const float* delta;     // [B, H, Sq]
  float* dq;              // [B, H, Sq, 128] fp32, zeroed
  int64_t dk_sb, dk_sh, dk_ss, dv_sb, dv_sh, dv_ss;
  int kv_blocks, q_blocks;
  int* status;
  // packed variable-length sequences (NULL: dense batch), as in the forward kernel; lse / delta are then [H, total_q]
  // and dq [H, total_q, 128]
  const int* cu_q;
  const int* cu_k;
  int total_q;
};

// adds a [128 rows x 32 floats] box of shared memory (128B-swizzled) into global memory at (x, y) of the tensor map
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                const __grid_constant__ CUtensorMap tmap_dq, T* __restrict__ dk, T* __restrict__ dv, const BwdParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sK = smem;
  uint8_t* sV = smem + kTile;
  uint8_t* sR = smem + 2 * kTile;                    // [kRing][kTile]: Q_i, dO_i, Q_{i+1}, ...
  uint8_t* sP = smem + (2 + kRing) * kTile;          // P^T  [keys x queries]
  uint8_t* sS = smem + (3 + kRing) * kTile;          // dS^T [keys x queries]
  float* s_lse = reinterpret_cast<float*>(smem + (4 + kRing) * kTile);   // [128]
  float* s_dlt = s_lse + 128;                                              // [128]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_dlt + 128);
  uint64_t* kv_full = bars;                  // 1
  uint64_t* r_full = bars + 1;               // [kRing]
  uint64_t* r_empty = r_full + kRing;        // [kRing]  tcgen05.commit
  uint64_t* s_full = r_empty + kRing;        // tcgen05.commit: S^T ready
  uint64_t* dp_full = s_full + 1;            // tcgen05.commit: dP^T ready
  uint64_t* s_free = dp_full + 1;            // 8 warps: S^T read
  uint64_t* p_ready = s_free + 1;            // 8 warps: P^T in shared memory
  uint64_t* ds_ready = p_ready + 1;          // 8 warps: dS^T in shared memory, dP^T read
  uint64_t* mma2_done = ds_ready + 1;        // tcgen05.commit: dV, dK, dQ of this pair complete
  uint64_t* dq_drained = mma2_done + 1;      // 8 warps: dQ read out of TMEM
  uint64_t* stage_free = dq_drained + 1;     // one thread: the TMA reduction has read the staged dQ
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(stage_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // all (batch, head) instances of the earliest key block first: under a causal mask it meets the most query blocks
  const int n_bh = p.B * p.Hkv;
  const int kb = (int)(blockIdx.x / n_bh);
  const int bh = (int)(blockIdx.x % n_bh);
  const int b = bh / p.Hkv, hk = bh - b * p.Hkv;
  const int G = p.H / p.Hkv;
  const int k0 = kb * BK;
  // this instance's sequence (see the forward kernel): rows past a packed sequence's end are loaded, masked by index
  // (their probabilities and score gradients are exact zeros) and never stored
  int Sq = p.Sq, Sk = p.Sk, qoff = 0, koff = 0, bt = b, q_blocks = p.q_blocks;
  if (p.cu_q) {
    qoff = p.cu_q[b];
    Sq = p.cu_q[b + 1] - qoff;
    koff = p.cu_k[b];
    Sk = p.cu_k[b + 1] - koff;
    bt = 0;
    q_blocks = (Sq + BQ - 1) / BQ;
  }
  const int i0 = p.causal ? min(q_blocks, k0 / BQ) : 0;   // first query block that sees these keys
  const int n_i = k0 < Sk ? q_blocks - i0 : 0;            // a key block past the sequence's end has nothing to do
  const int n_it = n_i * G;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(kv_full, 1);
    for (int s = 0; s < kRing; ++s) {
      mbar_init(&r_full[s], 1);
      mbar_init(&r_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(dp_full, 1);
    mbar_init(s_free, 8);
    mbar_init(p_ready, 8);
    mbar_init(ds_ready, 8);
    mbar_init(mma2_done, 1);
    mbar_init(dq_drained, 8);
    mbar_init(stage_free, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tmap_q);
    prefetch_tmap(&tmap_k);
    prefetch_tmap(&tmap_v);
    prefetch_tmap(&tmap_do);
    prefetch_tmap(&tmap_dq);
  }
  if (warp == 9) {
    tmem_alloc(tmem_slot, kBwdTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t kColS = 0, kColDP = 128, kColDV = 256, kColDK = 384;

  if (warp == 8) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0 && n_it > 0) {
      mbar_expect_tx(kv_full, 2 * kTile);
      tma_load_4d(sK, &tmap_k, kv_full, 0, koff + k0, hk, bt);
      tma_load_4d(sK + kTile / 2, &tmap_k, kv_full, 64, koff + k0, hk, bt);
      tma_load_4d(sV, &tmap_v, kv_full, 0, koff + k0, hk, bt);
      tma_load_4d(sV + kTile / 2, &tmap_v, kv_full, 64, koff + k0, hk, bt);
      for (int n = 0; n < 2 * n_it; ++n) {
        const int st = n % kRing;
        if (!mbar_wait(&r_empty[st], (uint32_t)(((n / kRing) & 1) ^ 1), abort_flag)) break;
        mbar_expect_tx(&r_full[st], kTile);
        const int it = n >> 1;
        const int h = hk * G + it / n_i;
        const int q0 = (i0 + it % n_i) * BQ;
        const CUtensorMap* map = (n & 1) ? &tmap_do : &tmap_q;
        tma_load_4d(sR + st * kTile, map, &r_full[st], 0, qoff + q0, h, bt);
        tma_load_4d(sR + st * kTile + kTile / 2, map, &r_full[st], 64, qoff + q0, h, bt);
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_it > 0) {
      const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      const uint32_t idesc_kk = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(128 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
      const uint32_t idesc_kmn = idesc_kk | (1u << 16);                 // B read MN-major
      const uint32_t idesc_mnmn = idesc_kk | (1u << 15) | (1u << 16);   // A and B read MN-major
      auto ring_wait = [&](int n) { return mbar_wait(&r_full[n % kRing], (uint32_t)((n / kRing) & 1), abort_flag); };
      // D = A B^T with both tiles K-major (two 64-column atoms, 32 bytes per k16 step)
      auto mma_kk = [&](uint32_t dcol, const uint8_t* a, const uint8_t* bt) {
        const uint32_t aa = smem_u32(a), ba = smem_u32(bt);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * (kTile / 2) + (uint32_t)(kk & 3) * 32;
          umma_f16(tmem_base + dcol, make_desc(aa + off, 16, 1024), make_desc(ba + off, 16, 1024), idesc_kk, kk != 0 ? 1u : 0u);
        }
      };
      // D (+)= A B with A K-major and B a [k rows x n columns] tile read MN-major (16 k rows = 2048 bytes per step)
      auto mma_kmn = [&](uint32_t dcol, const uint8_t* a, const uint8_t* bt, bool fresh) {
        const uint32_t aa = smem_u32(a), ba = smem_u32(bt);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t aoff = (uint32_t)(kk >> 2) * (kTile / 2) + (uint32_t)(kk & 3) * 32;
          umma_f16(tmem_base + dcol, make_desc(aa + aoff, 16, 1024), make_desc(ba + (uint32_t)kk * 2048, kTile / 2, 1024),
                   idesc_kmn, (fresh && kk == 0) ? 0u : 1u);
        }
      };
      // D = A^T B with A a [k rows x m columns] tile and B a [k rows x n columns] tile, both read MN-major
      auto mma_mnmn = [&](uint32_t dcol, const uint8_t* a, const uint8_t* bt) {
        const uint32_t aa = smem_u32(a), ba = smem_u32(bt);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_f16(tmem_base + dcol, make_desc(aa + (uint32_t)kk * 2048, kTile / 2, 1024),
                   make_desc(ba + (uint32_t)kk * 2048, kTile / 2, 1024), idesc_mnmn, kk != 0 ? 1u : 0u);
      };
      // Issue order per pair: dP^T, dV, then S^T of the NEXT pair (its TMEM columns are free once P^T has been formed, so
      // the tensor core computes it while the warpgroups still work on dS^T), then dK and dQ.
      bool ok = mbar_wait(kv_full, 0, abort_flag) && ring_wait(0);
      if (ok) {
        tc_fence_after();
        mma_kk(kColS, sK, sR);                         // S^T of the first pair (ring item 0)
        umma_commit(s_full);
      }
      for (int it = 0; it < n_it && ok; ++it) {
        const int nq = 2 * it, ndo = 2 * it + 1;
        const uint32_t par = (uint32_t)(it & 1), prev = par ^ 1u;
        const uint8_t* tQ = sR + (nq % kRing) * kTile;
        const uint8_t* tdO = sR + (ndo % kRing) * kTile;
        if (!ring_wait(ndo)) { ok = false; break; }
        if (it > 0 && !mbar_wait(dq_drained, prev, abort_flag)) { ok = false; break; }
        tc_fence_after();
        mma_kk(kColDP, sV, tdO);                     // dP^T = V dO^T
        umma_commit(dp_full);
        if (!mbar_wait(p_ready, par, abort_flag)) { ok = false; break; }
        tc_fence_after();
        mma_kmn(kColDV, sP, tdO, it == 0);           // dV += P^T dO
        if (it + 1 < n_it) {
          if (!ring_wait(nq + 2)) { ok = false; break; }
          if (!mbar_wait(s_free, par, abort_flag)) { ok = false; break; }
          tc_fence_after();
          mma_kk(kColS, sK, sR + ((nq + 2) % kRing) * kTile);   // S^T of the next pair
          umma_commit(s_full);
        }
        if (!mbar_wait(ds_ready, par, abort_flag)) { ok = false; break; }
        tc_fence_after();
        mma_kmn(kColDK, sS, tQ, it == 0);            // dK += dS^T Q
        mma_mnmn(kColDP, sS, sK);                    // dQ = dS K (over the consumed dP^T)
        umma_commit(mma2_done);
        umma_commit(&r_empty[nq % kRing]);
        umma_commit(&r_empty[ndo % kRing]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ two compute warpgroups (warps 0-3, 4-7)
    const int wg = warp >> 2;
    const int qw = warp & 3;
    const int r = qw * 32 + lane;                 // key row inside the block = TMEM lane
    const int kj = k0 + r;
    const uint32_t lane_base = ((uint32_t)(qw * 32) << 16);
    const int tid = threadIdx.x;                  // 0..255 here
    uint8_t* prow = sP + (size_t)wg * (kTile / 2) + (size_t)r * 128;   // this warpgroup's 64 query columns = atom `wg`
    uint8_t* srow = sS + (size_t)wg * (kTile / 2) + (size_t)r * 128;
    bool ok = true;
    auto wait_all = [&](uint64_t* bar, uint32_t parity) {
      const bool w = mbar_wait(bar, parity, abort_flag);
      return __all_sync(0xffffffffu, w);
    };
    for (int it = 0; it < n_it; ++it) {
      const uint32_t par = (uint32_t)(it & 1);
      const int h = hk * G + it / n_i;
      const int q0 = (i0 + it % n_i) * BQ;
      // lse (log2 domain) and delta (times the softmax scale) of the 128 query rows of this block; +inf switches a row
      // off.  Single buffers: a thread gets here only after mma2_done of the previous pair, which needs every warp's
      // ds_ready, i.e. all reads of the previous values.
      {
        const int which = tid >> 7, q = tid & 127, qi = q0 + q;
        const int64_t idx = p.cu_q ? (int64_t)h * p.total_q + qoff + qi : ((int64_t)b * p.H + h) * p.Sq + qi;
        if (which == 0) {
          float l = qi < Sq ? p.lse[idx] : -INFINITY;
          s_lse[q] = l > -INFINITY ? -l * 1.4426950408889634f : -INFINITY;   // negated: an addend of the exponent
        } else {
          s_dlt[q] = qi < Sq ? -p.delta[idx] * p.scale : 0.f;              // negated and scaled likewise
        }
      }
      named_bar_sync(1, 256);
      const float4* nlse4 = reinterpret_cast<const float4*>(s_lse + wg * 64);
      const float4* ndlt4 = reinterpret_cast<const float4*>(s_dlt + wg * 64);
      const bool diag = p.causal && q0 < k0 + BK;       // only then can a query be older than a key of this block
      const bool key_off = kj >= Sk;
      if (!wait_all(s_full, par)) { ok = false; break; }
      // the staged dQ of the previous pair must have left the shared memory that P^T is written to
      if (it > 0 && !wait_all(stage_free, par ^ 1u)) { ok = false; break; }
      tc_fence_after();
      float pf[64];
      {
        uint32_t ra[32], rb[32];
        auto chunk_p = [&](const uint32_t (&raw)[32], int c) {
          uint32_t pk[16];
#pragma unroll
          for (int e4 = 0; e4 < 8; ++e4) {
            const float4 nl = nlse4[c * 8 + e4];
            const float nls[4] = {nl.x, nl.y, nl.z, nl.w};
#pragma unroll
            for (int e2 = 0; e2 < 4; e2 += 2) {
              const int e = e4 * 4 + e2, cc = c * 32 + e;
              float x0, x1;
              fma2v(x0, x1, __uint_as_float(raw[e]), __uint_as_float(raw[e + 1]), p.scale_log2, nls[e2], nls[e2 + 1]);
              float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
              if (key_off || diag) {
                const int qi = q0 + wg * 64 + cc;
                if (key_off || qi < kj) p0 = 0.f;
                if (key_off || qi + 1 < kj) p1 = 0.f;
              }
              pf[cc] = p0;
              pf[cc + 1] = p1;
              pk[e >> 1] = pack2<T>(p0, p1);
            }
          }
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            const int ch = c * 4 + g8;
            *reinterpret_cast<uint4*>(prow + (size_t)((ch ^ (r & 7)) * 16)) =
                make_uint4(pk[g8 * 4], pk[g8 * 4 + 1], pk[g8 * 4 + 2], pk[g8 * 4 + 3]);
          }
        };
        const uint32_t addr = tmem_base + lane_base + kColS + (uint32_t)(wg * 64);
        tmem_ld32(addr, ra);
        tmem_ld_wait();
        tmem_ld32(addr + 32u, rb);
        chunk_p(ra, 0);
        tmem_ld_wait();
        chunk_p(rb, 1);
      }
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(s_free);
        mbar_arrive(p_ready);
      }
      if (!wait_all(dp_full, par)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t ra[32], rb[32];
        auto chunk_ds = [&](const uint32_t (&raw)[32], int c) {
          uint32_t pk[16];
#pragma unroll
          for (int e4 = 0; e4 < 8; ++e4) {
            const float4 nd = ndlt4[c * 8 + e4];
            const float nds[4] = {nd.x, nd.y, nd.z, nd.w};
#pragma unroll
            for (int e2 = 0; e2 < 4; e2 += 2) {
              const int e = e4 * 4 + e2, cc = c * 32 + e;
              float t0, t1, d0, d1;
              fma2v(t0, t1, __uint_as_float(raw[e]), __uint_as_float(raw[e + 1]), p.scale, nds[e2], nds[e2 + 1]);
              mul2(d0, d1, pf[cc], pf[cc + 1], t0, t1);
              pk[e >> 1] = pack2<T>(d0, d1);
            }
          }
#pragma unroll
          for (int g8 = 0; g8 < 4; ++g8) {
            const int ch = c * 4 + g8;
            *reinterpret_cast<uint4*>(srow + (size_t)((ch ^ (r & 7)) * 16)) =
                make_uint4(pk[g8 * 4], pk[g8 * 4 + 1], pk[g8 * 4 + 2], pk[g8 * 4 + 3]);
          }
        };
        const uint32_t addr = tmem_base + lane_base + kColDP + (uint32_t)(wg * 64);
        tmem_ld32(addr, ra);
        tmem_ld_wait();
        tmem_ld32(addr + 32u, rb);
        chunk_ds(ra, 0);
        tmem_ld_wait();
        chunk_ds(rb, 1);
      }
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_ready);
      // dQ of this pair: lane = query row, this warpgroup's 64 head-dim columns.  Staged as fp32 in the 64 KB that
      // P^T and dS^T occupied (the MMAs that read them have completed): four [128 rows x 128 bytes] boxes, 128B-swizzled.
      if (!wait_all(mma2_done, par)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t ra[32], rb[32];
        auto stage = [&](const uint32_t (&raw)[32], int c) {
          uint8_t* box = sP + (size_t)(wg * 2 + c) * (kTile / 2) + (size_t)r * 128;
#pragma unroll
          for (int ch = 0; ch < 8; ++ch)
            *reinterpret_cast<uint4*>(box + (size_t)((ch ^ (r & 7)) * 16)) =
                make_uint4(raw[ch * 4], raw[ch * 4 + 1], raw[ch * 4 + 2], raw[ch * 4 + 3]);
        };
        const uint32_t addr = tmem_base + lane_base + kColDP + (uint32_t)(wg * 64);
        tmem_ld32(addr, ra);
        tmem_ld_wait();
        tmem_ld32(addr + 32u, rb);
        stage(ra, 0);
        tmem_ld_wait();
        stage(rb, 1);
      }
      tc_fence_before();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_drained);
      named_bar_sync(2, 256);
      if (tid == 0) {
        const int row0 = p.cu_q ? (int)((int64_t)h * p.total_q + qoff + q0) : (int)(((int64_t)b * p.H + h) * p.Sq + q0);
#pragma unroll
        for (int c = 0; c < 4; ++c)
          tma_reduce_add_2d(&tmap_dq, sP + (size_t)c * (kTile / 2), c * 32, row0);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        mbar_arrive(stage_free);
      }
      __syncwarp();
    }
    // every reduction must have completed before the CTA exits
    if (tid == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    // ---- dK, dV of this key block (all pairs have completed: the last mma2_done was waited for above)
    if (ok) {
      tc_fence_after();
      const bool row_ok = kj < Sk;
      T* dk_row = dk + (int64_t)bt * p.dk_sb + (int64_t)hk * p.dk_sh + (int64_t)(koff + kj) * p.dk_ss + wg * 64;
      T* dv_row = dv + (int64_t)bt * p.dv_sb + (int64_t)hk * p.dv_sh + (int64_t)(koff + kj) * p.dv_ss + wg * 64;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t raw[32];
          if (n_it > 0) {
            tmem_ld32(tmem_base + lane_base + (which ? kColDK : kColDV) + (uint32_t)(wg * 64 + c * 32), raw);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) raw[e] = 0u;
          }
          if (row_ok) {
            T* dst = (which ? dk_row : dv_row) + c * 32;
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
              Vec16<T> v;
#pragma unroll
              for (int e = 0; e < 8; ++e) v.v[e] = ToF<T>::from(__uint_as_float(raw[g8 * 8 + e]));
              st16(dst + g8 * 8, v);
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kBwdTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
}

bool make_dq_map(CUtensorMap* out, float* ptr, int64_t rows) {
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
  if (!enc || rows <= 0) return false;
  cuuint64_t dims[2] = {128, (cuuint64_t)rows};
  cuuint64_t strides[1] = {128 * sizeof(float)};
  cuuint32_t box[2] = {32, 128};
  cuuint32_t estr[2] = {1, 1};
  return enc(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// delta[b, h, q] = sum_d O[b, h, q, d] * dO[b, h, q, d]; one warp per row
template <typename T>
__global__ void attn_delta_kernel(const T* __restrict__ o, const T* __restrict__ d_o, float* __restrict__ delta, int B,
                                  int H, int Sq, int64_t o_sb, int64_t o_sh, int64_t o_ss, int64_t g_sb, int64_t g_sh,
                                  int64_t g_ss) {
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= (int64_t)B * H * Sq) return;
  const int q = (int)(row % Sq);
  const int h = (int)((row / Sq) % H);
  const int b = (int)(row / ((int64_t)Sq * H));
  const T* po = o + b * o_sb + h * o_sh + q * o_ss + lane * 4;
  const T* pg = d_o + b * g_sb + h * g_sh + q * g_ss + lane * 4;
  const uint2 a = *reinterpret_cast<const uint2*>(po), g = *reinterpret_cast<const uint2*>(pg);
  const T* av = reinterpret_cast<const T*>(&a);
  const T* gv = reinterpret_cast<const T*>(&g);
  float s = 0.f;
#pragma unroll
  for (int e = 0; e < 4; ++e) s += ToF<T>::to(av[e]) * ToF<T>::to(gv[e]);
  s = warp_sum(s);
  if (lane == 0) delta[row] = s;
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int b200_flash_attn_bwd(const b200_attn_t* a, float* dq_accum, void* dk, void* dv, float* delta, const void* q,
                                   const void* k, const void* v, const void* o, const void* d_o, const float* lse,
                                   const int64_t* extra_strides, cudaStream_t stream) {
  // extra_strides: do_sb, do_sh, do_ss, dk_sb, dk_sh, dk_ss, dv_sb, dv_sh, dv_ss (elements)
  if (a->head_dim != BD || (a->dtype != B200_BF16 && a->dtype != B200_F16) || a->B <= 0 || a->H <= 0 || a->Hkv <= 0 ||
      a->H % a->Hkv != 0 || a->Sq <= 0 || a->Sk <= 0)
    return (int)cudaErrorNotSupported;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  const int64_t* x = extra_strides;
  const int64_t strides[] = {a->q_sb, a->q_sh, a->q_ss, a->k_sb, a->k_sh, a->k_ss, a->v_sb, a->v_sh, a->v_ss,
                             a->o_sb, a->o_sh, a->o_ss, x[0], x[1], x[2], x[3], x[4], x[5], x[6], x[7], x[8]};
  for (int64_t s : strides)
    if (s % 8 != 0) return (int)cudaErrorNotSupported;
  if (!al(q) || !al(k) || !al(v) || !al(o) || !al(d_o) || !al(dk) || !al(dv) || !al(dq_accum)) return (int)cudaErrorNotSupported;
  const bool packed = a->cu_seqlens_q != nullptr;
  if (packed && (!a->cu_seqlens_k || a->total_q <= 0 || a->total_k <= 0)) return (int)cudaErrorNotSupported;
  if ((a->B > 1 && !packed && (a->q_sb == 0 || a->k_sb == 0 || a->v_sb == 0 || x[0] == 0)) ||
      (a->H > 1 && (a->q_sh == 0 || x[1] == 0)) || (a->Hkv > 1 && (a->k_sh == 0 || a->v_sh == 0)) || a->q_ss == 0 ||
      a->k_ss == 0 || a->v_ss == 0 || x[2] == 0)
    return (int)cudaErrorNotSupported;
  const int bf16 = a->dtype == B200_BF16;
  CUtensorMap mq, mk, mv, mdo;
  auto nz = [](int64_t s, int64_t fallback) { return s ? s : fallback; };
  if (packed) {
    // one "batch" of total rows: the kernel adds each sequence's first row to its tile coordinates
    if (!make_attn_map(&mq, q, bf16, 1, a->H, a->total_q, (int64_t)a->total_q * a->q_ss, nz(a->q_sh, 8), a->q_ss) ||
        !make_attn_map(&mk, k, bf16, 1, a->Hkv, a->total_k, (int64_t)a->total_k * a->k_ss, nz(a->k_sh, 8), a->k_ss) ||
        !make_attn_map(&mv, v, bf16, 1, a->Hkv, a->total_k, (int64_t)a->total_k * a->v_ss, nz(a->v_sh, 8), a->v_ss) ||
        !make_attn_map(&mdo, d_o, bf16, 1, a->H, a->total_q, (int64_t)a->total_q * x[2], nz(x[1], 8), x[2]))
      return (int)cudaErrorNotSupported;
  } else if (!make_attn_map(&mq, q, bf16, a->B, a->H, a->Sq, nz(a->q_sb, 8), nz(a->q_sh, 8), a->q_ss) ||
             !make_attn_map(&mk, k, bf16, a->B, a->Hkv, a->Sk, nz(a->k_sb, 8), nz(a->k_sh, 8), a->k_ss) ||
             !make_attn_map(&mv, v, bf16, a->B, a->Hkv, a->Sk, nz(a->v_sb, 8), nz(a->v_sh, 8), a->v_ss) ||
             !make_attn_map(&mdo, d_o, bf16, a->B, a->H, a->Sq, nz(x[0], 8), nz(x[1], 8), x[2]))
    return (int)cudaErrorNotSupported;
  // dq_accum as a [B * H * Sq, 128] ([H * total_q, 128] when packed) fp32 matrix; one box = 32 columns of 128 rows
  const long long rows = packed ? (long long)a->H * a->total_q : (long long)a->B * a->H * a->Sq;
  const int dB = packed ? 1 : a->B, dS = packed ? a->total_q : a->Sq;     // the row-dot kernel's view of o and d_o
  CUtensorMap mdq;
  if (!make_dq_map(&mdq, dq_accum, rows)) return (int)cudaErrorNotSupported;
  BwdParams p{};
  p.B = a->B; p.H = a->H; p.Hkv = a->Hkv; p.Sq = a->Sq; p.Sk = a->Sk;
  p.causal = a->causal;
  p.scale = a->scale;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.lse = lse;
  p.delta = delta;
  p.dq = dq_accum;
  p.dk_sb = x[3]; p.dk_sh = x[4]; p.dk_ss = x[5];
  p.dv_sb = x[6]; p.dv_sh = x[7]; p.dv_ss = x[8];
  p.kv_blocks = (a->Sk + BK - 1) / BK;
  p.q_blocks = (a->Sq + BQ - 1) / BQ;
  p.status = gemm_status_word_device();
  p.cu_q = a->cu_seqlens_q;
  p.cu_k = a->cu_seqlens_k;
  p.total_q = a->total_q;
  const long long grid = (long long)a->B * a->Hkv * p.kv_blocks;
  if (grid > 2147483647ll || rows / 8 + 1 > 2147483647ll) return (int)cudaErrorNotSupported;
  cudaError_t e = cudaMemsetAsync(dq_accum, 0, (size_t)rows * BD * sizeof(float), stream);
  if (e != cudaSuccess) return (int)e;
  if (bf16) {
    attn_delta_kernel<__nv_bfloat16><<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(
        (const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, delta, dB, a->H, dS, a->o_sb, a->o_sh, a->o_ss, x[0], x[1], x[2]);
    static bool set = false;
    auto kern = attn_bwd_kernel<__nv_bfloat16>;
    if (!set) {
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem);
      if (e != cudaSuccess) return (int)e;
      set = true;
    }
    kern<<<(unsigned)grid, kBwdThreads, kBwdSmem, stream>>>(mq, mk, mv, mdo, mdq, (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, p);
  } else {
    attn_delta_kernel<__half><<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(
        (const __half*)o, (const __half*)d_o, delta, dB, a->H, dS, a->o_sb, a->o_sh, a->o_ss, x[0], x[1], x[2]);
    static bool set = false;
    auto kern = attn_bwd_kernel<__half>;
    if (!set) {
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kBwdSmem);
      if (e != cudaSuccess) return (int)e;
      set = true;
    }
    kern<<<(unsigned)grid, kBwdThreads, kBwdSmem, stream>>>(mq, mk, mv, mdo, mdq, (__half*)dk, (__half*)dv, p);
  }
  note_launch(2);
  return (int)cudaGetLastError();
}
