// Grouped bf16/fp16 GEMM on the 5th-generation tensor cores: G problems that share their shapes except for one
// ragged extent whose per-group lengths live in DEVICE memory (the rows a mixture-of-experts layer received for
// each of its experts), so that no host read of the counts sits between the token exchange and the expert GEMMs.
//
//   ragged rows   (forward, input gradient):  D[r, :] = A[r, :] * B[g(r)]^T     r in [off_g, off_g + count_g)
//       A [rows, K] and D [rows, N] are packed group after group; B is [G, N, K] (K-major) or [G, K, N] (MN-major).
//   ragged depth  (weight gradient):          D[g] = A[off_g : off_g + count_g, :]^T * B[off_g : off_g + count_g, :]
//       A [rows, M] and B [rows, N] are packed, both MN-major to the tensor core; D is [G, M, N].
//
// The machinery is that of the dense kernel: one persistent CTA per SM, 128x256 tiles, warp 0 = TMA producer
// (no multicast) into a 4-stage ring of 128-byte-swizzled tiles, warp 1 = tcgen05.mma issuer into one of two
// 256-column TMEM accumulators, warps 2-5 = tcgen05.ld epilogue.  What differs:
//   * every role derives the tile list from the counts (prefix sums in shared memory): row tiles never straddle
//     two groups' weights; a tile may load rows of the next group, its stores are limited to its own rows;
//   * with ragged depth the last 64-row block of a group overshoots into the next group's rows: after the TMA
//     data landed, the issuer warp overwrites those rows with zeros in shared memory (whole 128-byte swizzle rows,
//     so the swizzle does not matter) and fences the async proxy before the MMAs read the tile.
// Every mbarrier wait is bounded (status word as in the dense kernel).
//
// Parity: the reference multiplies experts one by one through its vendor GEMM
// (reference torch_musa/csrc/aten/ops/Matmul.cpp:293-335); it has no grouped entry point.
#include "gemm_common.cuh"

namespace b200k {
namespace {
using namespace gemmdev;

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kAccStages = 2;
constexpr int kThreads = 192;
constexpr int kATileBytes = BM * BK * 2;
constexpr int kBTileBytes = BN * BK * 2;
constexpr int kStageBytes = kATileBytes + kBTileBytes;
constexpr int kMaxGroups = 64;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256 + 2 * (kMaxGroups + 1) * 4;
constexpr uint32_t kTmemCols = 512;

struct GParams {
  int rows;        // packed rows (capacity of the packed operands)
  int m, n, k;     // ragged rows: n, k used; ragged depth: m, n used
  int groups;
  const int* counts;
  int tiles_m, tiles_n;   // ragged depth: tiles of one group's output
  int64_t ldd, stride_d;
  uint32_t idesc;
  int* status;
  int group_m;
};

// RAGGED_K = false: ragged rows (A K-major, B K-major or MN-major).  RAGGED_K = true: ragged depth (both MN-major).
template <typename OutT, bool RAGGED_K, bool B_KMAJOR>
__global__ void __launch_bounds__(kThreads, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    OutT* __restrict__ d, const GParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kATileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* tfull_bar = bars + 2 * kStages;
  uint64_t* tempty_bar = tfull_bar + kAccStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + kAccStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* s_off = reinterpret_cast<int*>(tmem_slot + 4);     // [groups + 1] first packed row of each group
  int* s_tile = s_off + (kMaxGroups + 1);                 // [groups + 1] first row tile of each group (ragged rows)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < kAccStages; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
    int off = 0, tile = 0;
    for (int g = 0; g < p.groups; ++g) {
      s_off[g] = off;
      s_tile[g] = tile;
      int c = p.counts[g];
      c = c < 0 ? 0 : c;
      if (c > p.rows - off) c = p.rows - off;
      off += c;
      tile += (c + BM - 1) / BM;
    }
    s_off[p.groups] = off;
    s_tile[p.groups] = tile;
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int tiles_per_group = p.tiles_m * p.tiles_n;                        // ragged depth
  const int total_tiles = RAGGED_K ? tiles_per_group * p.groups : s_tile[p.groups] * p.tiles_n;
  const int dense_kb = (p.k + BK - 1) / BK;                                 // ragged rows

  // tile -> (group, first output row, first output column, first depth row, depth blocks, rows of depth)
  auto locate = [&](int tile, int& g, int& m0, int& n0, int& krow0, int& kbs, int& kcount) {
    int mt, nt;
    if constexpr (RAGGED_K) {
      g = tile / tiles_per_group;
      decode_tile(tile - g * tiles_per_group, p.tiles_m, p.tiles_n, p.group_m, mt, nt);
      m0 = mt * BM;
      krow0 = s_off[g];
      kcount = s_off[g + 1] - s_off[g];
      kbs = (kcount + BK - 1) / BK;
    } else {
      decode_tile(tile, s_tile[p.groups], p.tiles_n, p.group_m, mt, nt);
      g = 0;
      while (g + 1 < p.groups && mt >= s_tile[g + 1]) ++g;
      m0 = s_off[g] + (mt - s_tile[g]) * BM;
      krow0 = 0;
      kcount = p.k;
      kbs = dense_kb;
    }
    n0 = nt * BN;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int g, m0, n0, krow0, kbs, kcount;
        locate(tile, g, m0, n0, krow0, kbs, kcount);
        for (int kb = 0; kb < kbs; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&full_bar[stage], kStageBytes);
          uint8_t* sa = smem_a + stage * kATileBytes;
          uint8_t* sb = smem_b + stage * kBTileBytes;
          const int k0 = krow0 + kb * BK;
          if constexpr (RAGGED_K) {
            tma_load_3d(sa, &tmap_a, &full_bar[stage], m0, k0, 0);
            tma_load_3d(sa + 8192, &tmap_a, &full_bar[stage], m0 + 64, k0, 0);
#pragma unroll
            for (int q = 0; q < 4; ++q) tma_load_3d(sb + q * 8192, &tmap_b, &full_bar[stage], n0 + q * 64, k0, 0);
          } else {
            tma_load_3d(sa, &tmap_a, &full_bar[stage], k0, m0, 0);
            if constexpr (B_KMAJOR) {
              tma_load_3d(sb, &tmap_b, &full_bar[stage], k0, n0, g);
            } else {
#pragma unroll
              for (int q = 0; q < 4; ++q) tma_load_3d(sb + q * 8192, &tmap_b, &full_bar[stage], n0 + q * 64, k0, g);
            }
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (whole warp waits; lane 0 issues)
    constexpr bool A_KMAJOR = !RAGGED_K;
    constexpr bool BK_MAJOR = !RAGGED_K && B_KMAJOR;
    int stage = 0, acc = 0;
    uint32_t phase = 0, acc_phase = 0;
    bool ok = true;
    // lane 0 waits, the warp takes its answer: the lanes can never disagree about leaving the loop
    auto warp_wait = [&](uint64_t* bar, uint32_t parity) {
      int w = 1;
      if (lane == 0) w = mbar_wait(bar, parity, abort_flag) ? 1 : 0;
      w = __shfl_sync(0xffffffffu, w, 0);
      __syncwarp();
      return w != 0;
    };
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      int g, m0, n0, krow0, kbs, kcount;
      locate(tile, g, m0, n0, krow0, kbs, kcount);
      if (!warp_wait(&tempty_bar[acc], acc_phase ^ 1)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
      for (int kb = 0; kb < kbs; ++kb) {
        if (!warp_wait(&full_bar[stage], phase)) { ok = false; break; }
        tc_fence_after();
        uint8_t* pa = smem_a + stage * kATileBytes;
        uint8_t* pb = smem_b + stage * kBTileBytes;
        if constexpr (RAGGED_K) {
          const int valid = kcount - kb * BK;          // depth rows of this block that belong to the group
          if (valid < BK) {
            // rows [valid, 64) of every 64-wide box are contiguous: (64 - valid) * 128 bytes at box + valid * 128
            const int n16 = (BK - valid) * 8;          // 16-byte words per box
            const uint4 z = make_uint4(0, 0, 0, 0);
            for (int box = 0; box < 6; ++box) {
              uint8_t* base = (box < 2 ? pa + box * 8192 : pb + (box - 2) * 8192) + valid * 128;
              for (int i = lane; i < n16; i += 32) reinterpret_cast<uint4*>(base)[i] = z;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          }
          __syncwarp();
        }
        if (lane == 0) {
          const uint32_t sa = smem_u32(pa);
          const uint32_t sb = smem_u32(pb);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t adesc = A_KMAJOR ? make_desc(sa + kk * 32, 16, 1024) : make_desc(sa + kk * 2048, 8192, 1024);
            const uint64_t bdesc = BK_MAJOR ? make_desc(sb + kk * 32, 16, 1024) : make_desc(sb + kk * 2048, 8192, 1024);
            umma_f16(tmem_d, adesc, bdesc, p.idesc, (kb > 0 || kk != 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1; }
      }
      if (!ok) break;
      if (lane == 0) umma_commit(&tfull_bar[acc]);
      __syncwarp();
      if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = (p.ldd % (16 / (int)sizeof(OutT)) == 0) && ((reinterpret_cast<uintptr_t>(d) & 15) == 0) &&
                        (p.stride_d % (16 / (int)sizeof(OutT)) == 0);
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      int g, m0, n0, krow0, kbs, kcount;
      locate(tile, g, m0, n0, krow0, kbs, kcount);
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) break;
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const int row_end = RAGGED_K ? p.m : s_off[g + 1];
      OutT* drow = d + (RAGGED_K ? (int64_t)g * p.stride_d : (int64_t)0) + (int64_t)row * p.ldd + n0;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.n) break;
        uint32_t raw[32];
        tmem_ld32(taddr + (uint32_t)(c * 32), raw);
        tmem_ld_wait();
        if (row < row_end) {
          const int valid = min(32, p.n - col0);
          float v[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = kbs > 0 ? __uint_as_float(raw[e]) : 0.f;   // an empty group: zeros
          store_chunk<OutT>(drow + c * 32, v, valid, vec_ok);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
}

template <typename OutT, bool RAGGED_K, bool B_KMAJOR>
int go(const CUtensorMap& ma, const CUtensorMap& mb, void* d, const GParams& p, int grid, cudaStream_t stream) {
  static bool attr_set = false;
  auto kern = grouped_gemm_kernel<OutT, RAGGED_K, B_KMAJOR>;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  kern<<<grid, kThreads, kSmemBytes, stream>>>(ma, mb, (OutT*)d, p);
  B200K_LAUNCH_RET();
}

template <typename OutT>
int launch(const b200_grouped_gemm_t* g, void* d, const void* a, const void* b, cudaStream_t stream) {
  CUtensorMap ma, mb;
  bool ok;
  GParams p{};
  p.rows = g->rows;
  p.m = g->m; p.n = g->n; p.k = g->k;
  p.groups = g->groups;
  p.counts = g->counts;
  p.ldd = g->ldd;
  p.stride_d = g->stride_d;
  p.status = gemm_status_word_device();
  const uint32_t fmt = g->in_dtype == B200_BF16 ? 1u : 0u;
  int upper_tiles;
  if (g->ragged_depth) {
    // A [rows, M] and B [rows, N]: MN-major boxes of 64 x 64
    ok = gemm_make_map(&ma, a, g->in_dtype, (uint64_t)g->m, (uint64_t)g->rows, 1, (uint64_t)g->lda * 2, 0, 64, BK) &&
         gemm_make_map(&mb, b, g->in_dtype, (uint64_t)g->n, (uint64_t)g->rows, 1, (uint64_t)g->ldb * 2, 0, 64, BK);
    p.tiles_m = (g->m + BM - 1) / BM;
    p.tiles_n = (g->n + BN - 1) / BN;
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(BN >> 3) << 17) |
              ((uint32_t)(BM >> 4) << 24);
    p.group_m = gemm_group_m(BM, g->m, g->rows / std::max(g->groups, 1), true);
    upper_tiles = p.tiles_m * p.tiles_n * g->groups;
  } else {
    ok = gemm_make_map(&ma, a, g->in_dtype, (uint64_t)g->k, (uint64_t)g->rows, 1, (uint64_t)g->lda * 2, 0, BK, BM);
    if (ok) {
      if (g->b_kmajor)
        ok = gemm_make_map(&mb, b, g->in_dtype, (uint64_t)g->k, (uint64_t)g->n, (uint64_t)g->groups,
                           (uint64_t)g->ldb * 2, (uint64_t)g->stride_b * 2, BK, BN);
      else
        ok = gemm_make_map(&mb, b, g->in_dtype, (uint64_t)g->n, (uint64_t)g->k, (uint64_t)g->groups,
                           (uint64_t)g->ldb * 2, (uint64_t)g->stride_b * 2, 64, BK);
    }
    p.tiles_m = 0;
    p.tiles_n = (g->n + BN - 1) / BN;
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((g->b_kmajor ? 0u : 1u) << 16) | ((uint32_t)(BN >> 3) << 17) |
              ((uint32_t)(BM >> 4) << 24);
    p.group_m = gemm_group_m(BM, g->rows, g->k, false);
    upper_tiles = ((g->rows + BM - 1) / BM + g->groups) * p.tiles_n;
  }
  if (!ok) return (int)cudaErrorNotSupported;
  const int grid = std::max(1, std::min(upper_tiles, gemm_sm_count()));
  if (g->ragged_depth) return go<OutT, true, false>(ma, mb, d, p, grid, stream);
  if (g->b_kmajor) return go<OutT, false, true>(ma, mb, d, p, grid, stream);
  return go<OutT, false, false>(ma, mb, d, p, grid, stream);
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int b200_grouped_gemm(const b200_grouped_gemm_t* g, void* d, const void* a, const void* b,
                                 cudaStream_t stream) {
  if (!g || !g->counts || g->groups <= 0 || g->groups > kMaxGroups || g->rows <= 0 || g->n <= 0) return (int)cudaErrorNotSupported;
  if (g->in_dtype != B200_BF16 && g->in_dtype != B200_F16) return (int)cudaErrorNotSupported;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al(a) || !al(b) || g->lda % 8 != 0 || g->ldb % 8 != 0) return (int)cudaErrorNotSupported;
  if (g->ragged_depth) {
    if (g->m < 8 || g->n < 8) return (int)cudaErrorNotSupported;
  } else {
    if (g->k < 8 || g->stride_b % 8 != 0 || (!g->b_kmajor && g->n < 8)) return (int)cudaErrorNotSupported;
  }
  switch (g->out_dtype) {
    case B200_BF16: return launch<__nv_bfloat16>(g, d, a, b, stream);
    case B200_F16: return launch<__half>(g, d, a, b, stream);
    case B200_F32: return launch<float>(g, d, a, b, stream);
    default: return (int)cudaErrorNotSupported;
  }
}
