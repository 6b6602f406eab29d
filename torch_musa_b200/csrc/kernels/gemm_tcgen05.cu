// bf16/fp16 GEMM on the 5th-generation tensor cores.
//
//   D[M,N] (+)= alpha * A[M,K] * B[N,K]^T (+ bias) (act)
//
// One persistent CTA per SM walks 128x256 output tiles.  Six warps, three roles:
//   warp 0   TMA producer: cp.async.bulk.tensor (no multicast) fills a 4-stage ring of
//            128x64 A and 256x64 B tiles in 128B-swizzled shared memory;
//   warp 1   MMA issuer: one elected lane issues tcgen05.mma (cta_group::1, kind::f16,
//            M128 N256 K16) from shared-memory descriptors into one of two 256-column
//            TMEM accumulators and releases ring slots with tcgen05.commit;
//   warps 2-5 epilogue: tcgen05.ld the finished accumulator (each warp its 32 TMEM lanes),
//            apply alpha / bias / activation / accumulate, convert, store 16-byte vectors.
// The two TMEM accumulators let the epilogue of tile i overlap the main loop of tile i+1.
// Either operand may be K-major or MN-major in memory (forward, dgrad and wgrad GEMMs
// without explicit transposes): MN-major tiles are fetched as 64-element boxes and
// described to the tensor core with the MN-major canonical layout.
// Every mbarrier wait is bounded: on expiry the CTA records a status word, stops issuing
// work, frees its TMEM and returns, so a broken pipeline can never hang the device.
//
// Parity: the reference sends mm/addmm/bmm to a closed vendor library
// (reference torch_musa/csrc/aten/ops/Matmul.cpp:293-335,373-380).
#include "gemm_common.cuh"

#include <cstdlib>
#include <mutex>
#include <unordered_map>

namespace b200k {
namespace {
using namespace gemmdev;

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kAccStages = 2;
constexpr int kThreads = 192;
constexpr int kATileBytes = BM * BK * 2;  // 16 KB
constexpr int kBTileBytes = BN * BK * 2;  // 32 KB
constexpr int kStageBytes = kATileBytes + kBTileBytes;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr uint32_t kTmemCols = 512;

// TF32: fp32 operands (K-major only), 32 elements = 128 bytes per K block, kind::tf32.
template <typename OutT, bool A_KMAJOR, bool B_KMAJOR, bool TF32 = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, OutT* __restrict__ d,
            const Params p) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment is required by the 128-byte swizzle atoms.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kStages * kATileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* full_bar = bars;                       // [kStages]
  uint64_t* empty_bar = bars + kStages;            // [kStages]
  uint64_t* tfull_bar = bars + 2 * kStages;        // [kAccStages]
  uint64_t* tempty_bar = tfull_bar + kAccStages;   // [kAccStages]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + kAccStages);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int BKE = TF32 ? 32 : BK;  // elements per K block (always 128 bytes)
  const int k_blocks = (p.k + BKE - 1) / BKE;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int tiles_all_batches = tiles_per_batch * p.batch;
  const int total_tiles = tiles_all_batches * p.splits;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int s = 0; s < kAccStages; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], 4);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int split = tile / tiles_all_batches;
        const int tb = tile - split * tiles_all_batches;
        const int b = tb / tiles_per_batch;
        const int r = tb - b * tiles_per_batch;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(k_blocks, kb0 + p.kb_per_split);
        int mt, nt;
        decode_tile(r, p.tiles_m, p.tiles_n, p.group_m, mt, nt);
        const int m0 = mt * BM;
        const int n0 = nt * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&full_bar[stage], kStageBytes);
          uint8_t* sa = smem_a + stage * kATileBytes;
          uint8_t* sb = smem_b + stage * kBTileBytes;
          const int k0 = kb * BKE;
          if constexpr (A_KMAJOR) {
            tma_load_3d(sa, &tmap_a, &full_bar[stage], k0, m0, b);
          } else {
            // MN-major: two 64(M) x 64(K) boxes, 8 KB each
            tma_load_3d(sa, &tmap_a, &full_bar[stage], m0, k0, b);
            tma_load_3d(sa + 8192, &tmap_a, &full_bar[stage], m0 + 64, k0, b);
          }
          if constexpr (B_KMAJOR) {
            tma_load_3d(sb, &tmap_b, &full_bar[stage], k0, n0, b);
          } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) tma_load_3d(sb + q * 8192, &tmap_b, &full_bar[stage], n0 + q * 64, k0, b);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int kb0 = (tile / tiles_all_batches) * p.kb_per_split;
        const int kb1 = min(k_blocks, kb0 + p.kb_per_split);
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem_a + stage * kATileBytes);
          const uint32_t sb = smem_u32(smem_b + stage * kBTileBytes);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            // K-major: 16 elements = 32 B inside the 128-byte swizzle row; SBO = 8 rows x 128 B.
            // MN-major: 16 k-rows of 128 B = 2048 B; LBO = next 64-wide MN box (8 KB), SBO = 8 k-rows.
            const uint64_t adesc = A_KMAJOR ? make_desc(sa + kk * 32, 16, 1024) : make_desc(sa + kk * 2048, 8192, 1024);
            const uint64_t bdesc = B_KMAJOR ? make_desc(sb + kk * 32, 16, 1024) : make_desc(sb + kk * 2048, 8192, 1024);
            if constexpr (TF32) umma_tf32(tmem_d, adesc, bdesc, p.idesc, (kb > kb0 || kk != 0) ? 1u : 0u);
            else umma_f16(tmem_d, adesc, bdesc, p.idesc, (kb > kb0 || kk != 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);  // slot reusable once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);  // accumulator complete
        if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = (p.ldd % (16 / (int)sizeof(OutT)) == 0) && ((reinterpret_cast<uintptr_t>(d) & 15) == 0) &&
                        (p.stride_d % (16 / (int)sizeof(OutT)) == 0);
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      const int split = tile / tiles_all_batches;
      const int tb = tile - split * tiles_all_batches;
      const int b = tb / tiles_per_batch;
      const int r = tb - b * tiles_per_batch;
      int mt, nt;
      decode_tile(r, p.tiles_m, p.tiles_n, p.group_m, mt, nt);
      const int m0 = mt * BM;
      const int n0 = nt * BN;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, abort_flag)) break;
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      OutT* drow = d + (int64_t)split * p.split_stride + (int64_t)b * p.stride_d + (int64_t)row * p.ldd + n0;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.n) break;  // uniform across the warp
        uint32_t raw[32];
        tmem_ld32(taddr + (uint32_t)(c * 32), raw);
        tmem_ld_wait();
        if (row < p.m) {
          const int valid = min(32, p.n - col0);
          float v[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(raw[e]) * p.alpha;
          if (p.bias) {
            if (p.bias_f32) {
              const float* bp = reinterpret_cast<const float*>(p.bias) + col0;
#pragma unroll
              for (int e = 0; e < 32; ++e) if (e < valid) v[e] += __ldg(bp + e);
            } else {
              const OutT* bp = reinterpret_cast<const OutT*>(p.bias) + col0;
#pragma unroll
              for (int e = 0; e < 32; ++e) if (e < valid) v[e] += ToF<OutT>::to(bp[e]);
            }
          }
          if (p.act) {
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = apply_act(v[e], p.act);
          }
          if (p.accumulate) {
#pragma unroll
            for (int e = 0; e < 32; ++e) if (e < valid) v[e] += ToF<OutT>::to(drow[c * 32 + e]);
          }
          store_chunk<OutT>(drow + c * 32, v, valid, vec_ok);
        }
      }
      // all TMEM reads of this accumulator are complete (wait::ld above): hand it back
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

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess) {
      (void)cudaGetLastError();
      return (EncodeTiledFn) nullptr;
    }
    return (EncodeTiledFn)p;
  }();
  return fn;
}

struct MapKey {
  const void* ptr;
  uint64_t d0, d1, d2, s1, s2;
  uint32_t b0, b1;
  int dtype;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && s1 == o.s1 && s2 == o.s2 && b0 == o.b0 &&
           b1 == o.b1 && dtype == o.dtype;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    uint64_t h = (uint64_t)(uintptr_t)k.ptr * 0x9E3779B97F4A7C15ull;
    h ^= k.d0 + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.d1 + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= k.s1 + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= ((uint64_t)k.b0 << 32 | k.b1) + (h << 6) + (h >> 2);
    h ^= k.d2 * 31 + k.s2 * 17 + (uint64_t)k.dtype;
    return (size_t)h;
  }
};

// dims innermost-first: {inner, outer, batch}; strides in bytes for outer and batch; box {b0, b1, 1}
bool make_map(CUtensorMap* out, const void* ptr, int dtype, uint64_t inner, uint64_t outer, uint64_t batch,
              uint64_t outer_stride_bytes, uint64_t batch_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{ptr, inner, outer, batch, outer_stride_bytes, batch_stride_bytes, box_inner, box_outer, dtype};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  EncodeTiledFn enc = get_encode();
  if (!enc) return false;
  cuuint64_t dims[3] = {inner, outer, batch};
  cuuint64_t strides[2] = {outer_stride_bytes, batch_stride_bytes ? batch_stride_bytes : outer_stride_bytes * outer};
  cuuint32_t box[3] = {box_inner, box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMapDataType dt = dtype == B200_BF16  ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : dtype == B200_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  // experiment knob: L2 promotion size of the operand maps (0 none, 1 64 B, 2 128 B, 3 256 B = default)
  static const int promo = [] {
    const char* e = std::getenv("B200_GEMM_L2_PROMOTION");
    return e ? std::atoi(e) : 3;
  }();
  const CUtensorMapL2promotion pr = promo == 0   ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                                    : promo == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                                    : promo == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                                 : CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
  CUresult r = enc(out, dt, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, pr, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return true;
}

int* status_word() {
  // One pinned, device-mapped word per process: kernels write it only when a bounded wait expired.
  static int* host = [] {
    int* p = nullptr;
    if (cudaHostAlloc((void**)&p, sizeof(int), cudaHostAllocMapped) != cudaSuccess) {
      (void)cudaGetLastError();
      return (int*)nullptr;
    }
    *p = 0;
    return p;
  }();
  return host;
}

template <typename OutT>
int launch(const b200_gemm_desc_t* g, void* d, const void* a, const void* b, cudaStream_t stream,
           const GemmPlan& plan) {
  CUtensorMap ma, mb;
  const bool tf32 = g->in_dtype == B200_F32;
  const uint64_t esz = tf32 ? 4 : 2;
  const uint32_t BKH = tf32 ? 32 : BK;  // elements per 128-byte K block
  const uint64_t batch = (uint64_t)std::max(g->batch, 1);
  bool ok;
  if (tf32 && !(g->a_kmajor && g->b_kmajor)) return (int)cudaErrorNotSupported;
  if (g->a_kmajor)
    ok = make_map(&ma, a, g->in_dtype, (uint64_t)g->k, (uint64_t)g->m, batch, (uint64_t)g->lda * esz,
                  (uint64_t)g->stride_a * esz, BKH, BM);
  else
    ok = make_map(&ma, a, g->in_dtype, (uint64_t)g->m, (uint64_t)g->k, batch, (uint64_t)g->lda * esz,
                  (uint64_t)g->stride_a * esz, 64, BK);
  if (!ok) return (int)cudaErrorNotSupported;
  if (g->b_kmajor)
    ok = make_map(&mb, b, g->in_dtype, (uint64_t)g->k, (uint64_t)g->n, batch, (uint64_t)g->ldb * esz,
                  (uint64_t)g->stride_b * esz, BKH, BN);
  else
    ok = make_map(&mb, b, g->in_dtype, (uint64_t)g->n, (uint64_t)g->k, batch, (uint64_t)g->ldb * esz,
                  (uint64_t)g->stride_b * esz, 64, BK);
  if (!ok) return (int)cudaErrorNotSupported;

  Params p;
  p.m = g->m; p.n = g->n; p.k = g->k;
  p.batch = (int)batch;
  p.tiles_m = (g->m + BM - 1) / BM;
  p.tiles_n = (g->n + BN - 1) / BN;
  p.ldd = g->ldd;
  p.stride_d = g->stride_d;
  p.bias = g->bias;
  p.bias_f32 = g->bias_dtype == B200_F32;
  p.act = g->act;
  p.accumulate = g->accumulate;
  p.alpha = g->alpha;
  // instruction descriptor: fp32 accumulate, A/B format, majors, N>>3, M>>4
  const uint32_t fmt = g->in_dtype == B200_BF16 ? 1u : (g->in_dtype == B200_F32 ? 2u : 0u);  // f16 0, bf16 1, tf32 2
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((g->a_kmajor ? 0u : 1u) << 15) | ((g->b_kmajor ? 0u : 1u) << 16) |
            ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  int* host_status = status_word();
  int* dev_status = nullptr;
  if (host_status) {
    if (cudaHostGetDevicePointer((void**)&dev_status, host_status, 0) != cudaSuccess) {
      (void)cudaGetLastError();
      dev_status = nullptr;
    }
  }
  p.status = dev_status;
  p.splits = plan.splits;
  p.kb_per_split = plan.kb_per_split;
  p.split_stride = (int64_t)g->m * g->n;
  p.group_m = gemm_group_m(BM, g->m, plan.splits > 1 ? plan.kb_per_split * BK : g->k, !g->a_kmajor && !g->b_kmajor);

  const int total = p.tiles_m * p.tiles_n * p.batch * p.splits;
  int dev = 0, sms = kSMs;
  cudaGetDevice(&dev);
  static int cached_sms[64] = {0};
  if (dev < 64) {
    if (!cached_sms[dev]) cudaDeviceGetAttribute(&cached_sms[dev], cudaDevAttrMultiProcessorCount, dev);
    if (cached_sms[dev] > 0) sms = cached_sms[dev];
  }
  const int grid = std::min(total, sms);

#define GEMM_GO(AK, BKM)                                                                                         \
  do {                                                                                                           \
    static bool attr_set = false;                                                                                \
    auto kern = gemm_kernel<OutT, AK, BKM>;                                                                      \
    if (!attr_set) {                                                                                             \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);       \
      if (e != cudaSuccess) return (int)e;                                                                       \
      attr_set = true;                                                                                           \
    }                                                                                                            \
    kern<<<grid, kThreads, kSmemBytes, stream>>>(ma, mb, (OutT*)d, p);                                           \
  } while (0)

  if (tf32) {
    if constexpr (std::is_same<OutT, float>::value) {
      static bool attr_set = false;
      auto kern = gemm_kernel<float, true, true, true>;
      if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
      }
      kern<<<grid, kThreads, kSmemBytes, stream>>>(ma, mb, (float*)d, p);
      B200K_LAUNCH_RET();
    } else {
      return (int)cudaErrorNotSupported;
    }
  }
  if (g->a_kmajor && g->b_kmajor) GEMM_GO(true, true);
  else if (g->a_kmajor && !g->b_kmajor) GEMM_GO(true, false);
  else if (!g->a_kmajor && g->b_kmajor) GEMM_GO(false, true);
  else GEMM_GO(false, false);
#undef GEMM_GO
  B200K_LAUNCH_RET();
}

}  // namespace

bool gemm_make_map(CUtensorMap* out, const void* ptr, int dtype, uint64_t inner, uint64_t outer, uint64_t batch,
                   uint64_t outer_stride_bytes, uint64_t batch_stride_bytes, uint32_t box_inner, uint32_t box_outer) {
  return make_map(out, ptr, dtype, inner, outer, batch, outer_stride_bytes, batch_stride_bytes, box_inner, box_outer);
}
int* gemm_status_word_device() {
  int* host = status_word();
  int* dev = nullptr;
  if (host && cudaHostGetDevicePointer((void**)&dev, host, 0) != cudaSuccess) {
    (void)cudaGetLastError();
    dev = nullptr;
  }
  return dev;
}
int gemm_sm_count() {
  int dev = 0, sms = kSMs;
  cudaGetDevice(&dev);
  static int cached[64] = {0};
  if (dev >= 0 && dev < 64) {
    if (!cached[dev]) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
    if (cached[dev] > 0) sms = cached[dev];
  }
  return sms;
}
}  // namespace b200k

using namespace b200k;

extern "C" {

int b200_gemm_available(void) { return get_encode() != nullptr ? 1 : 0; }

// Non-zero once any GEMM launch of this process gave up on a bounded wait (sticky until cleared).
int b200_gemm_status(int clear) {
  int* s = status_word();
  if (!s) return 0;
  int v = *(volatile int*)s;
  if (clear) *(volatile int*)s = 0;
  return v;
}

static int gemm_validate(const b200_gemm_desc_t* g, const void* a, const void* b) {
  if (g->k <= 0) return (int)cudaErrorNotSupported;
  if (g->in_dtype != B200_BF16 && g->in_dtype != B200_F16 && g->in_dtype != B200_F32) return (int)cudaErrorNotSupported;
  if (g->in_dtype == B200_F32 && (!g->a_kmajor || !g->b_kmajor || g->out_dtype != B200_F32)) return (int)cudaErrorNotSupported;
  // TMA: base 16-byte aligned, byte strides multiples of 16
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (!al(a) || !al(b) || g->lda % 8 != 0 || g->ldb % 8 != 0) return (int)cudaErrorNotSupported;
  if (g->batch > 1 && (g->stride_a % 8 != 0 || g->stride_b % 8 != 0)) return (int)cudaErrorNotSupported;
  // a zero batch stride (broadcast operand) cannot be expressed as a tensor-map stride
  if (g->batch > 1 && (g->stride_a == 0 || g->stride_b == 0)) return (int)cudaErrorNotSupported;
  // the contiguous extent must cover at least one 16-byte unit
  if ((g->a_kmajor ? g->k : g->m) < 8 || (g->b_kmajor ? g->k : g->n) < 8) return (int)cudaErrorNotSupported;
  if (g->out_dtype != B200_BF16 && g->out_dtype != B200_F16 && g->out_dtype != B200_F32) return (int)cudaErrorNotSupported;
  return 0;
}

static int gemm_dispatch(const b200_gemm_desc_t* g, void* d, const void* a, const void* b, cudaStream_t stream,
                         const GemmPlan& plan) {
  if (plan.pair) return gemm_launch_2cta(g, d, a, b, stream, plan);
  switch (g->out_dtype) {
    case B200_BF16: return launch<__nv_bfloat16>(g, d, a, b, stream, plan);
    case B200_F16: return launch<__half>(g, d, a, b, stream, plan);
    case B200_F32: return launch<float>(g, d, a, b, stream, plan);
    default: return (int)cudaErrorNotSupported;
  }
}

// Bytes of fp32 scratch a split-K run of this problem wants (0: the problem is not split).  A caller that
// passes less in desc->workspace simply gets the unsplit kernel.
size_t b200_gemm_workspace_bytes(const b200_gemm_desc_t* g) {
  if (g->m <= 0 || g->n <= 0 || g->k <= 0) return 0;
  const GemmPlan plan = gemm_plan(g);
  return plan.splits > 1 ? (size_t)plan.splits * (size_t)g->m * (size_t)g->n * sizeof(float) : 0;
}

int b200_gemm(const b200_gemm_desc_t* g, void* d, const void* a, const void* b, cudaStream_t stream) {
  if (g->m <= 0 || g->n <= 0 || std::max(g->batch, 1) <= 0) return 0;
  int v = gemm_validate(g, a, b);
  if (v != 0) return v;
  GemmPlan plan = gemm_plan(g);
  if (plan.splits > 1) {
    const size_t need = (size_t)plan.splits * (size_t)g->m * (size_t)g->n * sizeof(float);
    if (g->workspace && g->workspace_bytes >= need && (reinterpret_cast<uintptr_t>(g->workspace) & 15) == 0) {
      // every split writes its fp32 partial product; one pass sums them and applies the epilogue
      b200_gemm_desc_t part = *g;
      part.out_dtype = B200_F32;
      part.ldd = g->n;
      part.stride_d = 0;
      part.bias = nullptr;
      part.act = 0;
      part.accumulate = 0;
      int e = gemm_dispatch(&part, g->workspace, a, b, stream, plan);
      if (e != 0) return e;
      return gemm_splitk_reduce(g, d, (const float*)g->workspace, plan.splits, stream);
    }
    plan.splits = 1;
    plan.kb_per_split = (g->k + BK - 1) / BK;
  }
  return gemm_dispatch(g, d, a, b, stream, plan);
}

}  // extern "C"
