// Block-scaled fp8 (e4m3 / e5m2) GEMM on the 5th-generation tensor cores.
//
//   D[M,N] = sum over 128-wide K blocks kb of  sa[m, kb] * sb[n / 128, kb] * (A[m, kb] . B[n, kb])   (* ra[m] * rb[n]) (+ bias)
//
// A [M,K] and B [N,K] are fp8, K contiguous.  One CTA owns a 128x128 output tile.  Warp 0 feeds a 5-stage ring of
// 128x128-byte A and B tiles with TMA (128-byte swizzle); warp 1 issues tcgen05.mma kind::f8f6f4 (M128 N128 K32, four
// per K block) into one of two 128-column TMEM accumulators, a fresh accumulation per K block; warps 2-5 promote:
// they read the finished block product from TMEM, multiply it by the block's two scale factors and add it to fp32
// accumulators in registers (each thread owns one output row), while the tensor core already works on the next
// block in the other TMEM accumulator.  The epilogue applies optional per-row / per-column factors (row-wise and
// tensor-wise scaling are the special case of block factors 1) and the bias, and stores bf16 / fp16 / fp32.
// Every mbarrier wait is bounded.
//
// Parity: the reference forwards _scaled_mm to its vendor library (reference torch_musa/csrc/aten/ops/Matmul.cpp:670-681).
#include "gemm_common.cuh"

#include <cuda_fp8.h>

#include <algorithm>

namespace b200k {
namespace {
using namespace gemmdev;

constexpr int FM = 128, FN = 128, FK = 128;     // tile; FK fp8 elements = 128 bytes = one swizzle row
constexpr int kF8Stages = 5;
constexpr int kF8Tile = FM * FK;                 // 16 KB per operand tile
constexpr int kF8Stage = 2 * kF8Tile;
constexpr int kF8Smem = kF8Stages * kF8Stage + 1024 + 256;
constexpr int kF8Threads = 192;
constexpr uint32_t kF8TmemCols = 256;            // two 128-column accumulators

struct F8Params {
  int m, n, k;
  int64_t ldd;
  const float* sa; int64_t sa_sm, sa_sk;         // block scales of A: sa[m * sa_sm + kb * sa_sk]   (NULL: 1)
  const float* sb; int64_t sb_sn, sb_sk;         // block scales of B: sb[(n / 128) * sb_sn + kb * sb_sk] (NULL: 1)
  const float* ra; int64_t ra_s;                 // final per-row factor ra[m * ra_s] (NULL: 1; ra_s 0: one scalar)
  const float* rb; int64_t rb_s;                 // final per-column factor rb[n * rb_s]
  const void* bias; int bias_f32;
  uint32_t idesc;
  int* status;
};

__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <typename OutT>
__global__ void __launch_bounds__(kF8Threads, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                OutT* __restrict__ d, const F8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + kF8Stages * kF8Tile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kF8Stages * kF8Stage);
  uint64_t* full_bar = bars;                  // [stages]
  uint64_t* empty_bar = bars + kF8Stages;     // [stages]
  uint64_t* tfull_bar = bars + 2 * kF8Stages; // [2]
  uint64_t* tempty_bar = tfull_bar + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_blocks = (p.k + FK - 1) / FK;
  const int tiles_m = (p.m + FM - 1) / FM;
  const int m0 = (blockIdx.x % tiles_m) * FM;
  const int n0 = (blockIdx.x / tiles_m) * FN;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kF8Stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&tfull_bar[s], 1); mbar_init(&tempty_bar[s], 4); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kF8TmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < k_blocks; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) break;
        mbar_expect_tx(&full_bar[stage], kF8Stage);
        tma_load_3d(smem_a + stage * kF8Tile, &tmap_a, &full_bar[stage], kb * FK, m0, 0);
        tma_load_3d(smem_b + stage * kF8Tile, &tmap_b, &full_bar[stage], kb * FK, n0, 0);
        if (++stage == kF8Stages) { stage = 0; phase ^= 1; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < k_blocks; ++kb) {
        const int slot = kb & 1;
        // the promotion warps must have drained this accumulator (block kb - 2)
        if (!mbar_wait(&tempty_bar[slot], (uint32_t)(((kb >> 1) & 1) ^ 1), abort_flag)) break;
        if (!mbar_wait(&full_bar[stage], phase, abort_flag)) break;
        tc_fence_after();
        const uint32_t sa = smem_u32(smem_a + stage * kF8Tile), sb = smem_u32(smem_b + stage * kF8Tile);
        const uint32_t tmem_d = tmem_base + (uint32_t)(slot * FN);
#pragma unroll
        for (int kk = 0; kk < FK / 32; ++kk)
          umma_f8(tmem_d, make_desc(sa + kk * 32, 16, 1024), make_desc(sb + kk * 32, 16, 1024), p.idesc, kk != 0 ? 1u : 0u);
        umma_commit(&empty_bar[stage]);
        umma_commit(&tfull_bar[slot]);
        if (++stage == kF8Stages) { stage = 0; phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ promotion + epilogue (warps 2..5)
    const int q = warp & 3;
    const int row = m0 + q * 32 + lane;
    const bool row_ok = row < p.m;
    float acc[FN];
#pragma unroll
    for (int c = 0; c < FN; ++c) acc[c] = 0.f;
    const float* sa_row = p.sa ? p.sa + (int64_t)min(row, p.m - 1) * p.sa_sm : nullptr;
    const float* sb_blk = p.sb ? p.sb + (int64_t)(n0 / FN) * p.sb_sn : nullptr;
    bool ok = true;
    for (int kb = 0; kb < k_blocks; ++kb) {
      const int slot = kb & 1;
      if (!mbar_wait(&tfull_bar[slot], (uint32_t)((kb >> 1) & 1), abort_flag)) { ok = false; break; }
      tc_fence_after();
      const float f = (sa_row ? sa_row[(int64_t)kb * p.sa_sk] : 1.f) * (sb_blk ? sb_blk[(int64_t)kb * p.sb_sk] : 1.f);
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(slot * FN);
#pragma unroll
      for (int c = 0; c < FN / 32; ++c) {
        uint32_t raw[32];
        tmem_ld32(taddr + (uint32_t)(c * 32), raw);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) acc[c * 32 + e] = fmaf(__uint_as_float(raw[e]), f, acc[c * 32 + e]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty_bar[slot]);
    }
    if (ok && row_ok) {
      const float fr = p.ra ? p.ra[(int64_t)row * p.ra_s] : 1.f;
      OutT* drow = d + (int64_t)row * p.ldd + n0;
      const bool vec_ok = (p.ldd % (16 / (int)sizeof(OutT)) == 0) && ((reinterpret_cast<uintptr_t>(d) & 15) == 0);
#pragma unroll
      for (int c = 0; c < FN / 32; ++c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.n) break;
        const int valid = min(32, p.n - col0);
        float v[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float x = acc[c * 32 + e] * fr;
          if (p.rb && e < valid) x *= p.rb[(int64_t)(col0 + e) * p.rb_s];
          if (p.bias && e < valid)
            x += p.bias_f32 ? reinterpret_cast<const float*>(p.bias)[col0 + e]
                            : ToF<OutT>::to(reinterpret_cast<const OutT*>(p.bias)[col0 + e]);
          v[e] = x;
        }
        store_chunk<OutT>(drow + c * 32, v, valid, vec_ok);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kF8TmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool make_u8_map(CUtensorMap* out, const void* ptr, uint64_t k, uint64_t rows, uint64_t ld_bytes) {
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
  cuuint64_t dims[3] = {k, rows, 1};
  cuuint64_t strides[2] = {ld_bytes, ld_bytes * rows};
  cuuint32_t box[3] = {FK, FM, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename OutT>
int launch_fp8(const b200_fp8_gemm_t* g, void* d, const void* a, const void* b, cudaStream_t stream) {
  CUtensorMap ma, mb;
  if (!make_u8_map(&ma, a, (uint64_t)g->k, (uint64_t)g->m, (uint64_t)g->lda) ||
      !make_u8_map(&mb, b, (uint64_t)g->k, (uint64_t)g->n, (uint64_t)g->ldb))
    return (int)cudaErrorNotSupported;
  F8Params p{};
  p.m = g->m; p.n = g->n; p.k = g->k;
  p.ldd = g->ldd;
  p.sa = g->block_scale_a; p.sa_sm = g->bsa_stride_m; p.sa_sk = g->bsa_stride_kb;
  p.sb = g->block_scale_b; p.sb_sn = g->bsb_stride_nb; p.sb_sk = g->bsb_stride_kb;
  p.ra = g->row_scale; p.ra_s = g->row_scale_stride;
  p.rb = g->col_scale; p.rb_s = g->col_scale_stride;
  p.bias = g->bias; p.bias_f32 = g->bias_dtype == B200_F32;
  // kind::f8f6f4 instruction descriptor: fp32 accumulate, operand formats (0 = e4m3, 1 = e5m2), K-major, N>>3, M>>4
  const uint32_t fa = g->a_e5m2 ? 1u : 0u, fb = g->b_e5m2 ? 1u : 0u;
  p.idesc = (1u << 4) | (fa << 7) | (fb << 10) | ((uint32_t)(FN >> 3) << 17) | ((uint32_t)(FM >> 4) << 24);
  p.status = gemm_status_word_device();
  static bool attr_set = false;
  auto kern = gemm_fp8_kernel<OutT>;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kF8Smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int grid = ((g->m + FM - 1) / FM) * ((g->n + FN - 1) / FN);
  kern<<<grid, kF8Threads, kF8Smem, stream>>>(ma, mb, (OutT*)d, p);
  B200K_LAUNCH_RET();
}

// ---- 1 x 128 block quantisation of activations: one warp per 128-element block
template <typename T>
__global__ void quant_1x128_kernel(const T* __restrict__ x, uint8_t* __restrict__ q, float* __restrict__ scales,
                                   int64_t rows, int k, int64_t ldx, int e5m2) {
  const int kblocks = k / 128;
  const int64_t nblk = rows * kblocks;
  const int lane = threadIdx.x & 31;
  const float fmax = e5m2 ? 57344.f : 448.f;
  for (int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < nblk; b += (int64_t)gridDim.x * (blockDim.x >> 5)) {
    const int64_t r = b / kblocks;
    const int kb = (int)(b - r * kblocks);
    const T* src = x + r * ldx + kb * 128 + lane * 4;
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = ToF<T>::to(src[i]);
    float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
    amax = warp_max(amax);
    const float scale = amax > 0.f ? amax / fmax : 1.f;
    const float inv = 1.f / scale;
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float y = fminf(fmaxf(v[i] * inv, -fmax), fmax);
      const __nv_fp8_storage_t f8 = __nv_cvt_float_to_fp8(y, __NV_SATFINITE, e5m2 ? __NV_E5M2 : __NV_E4M3);
      packed |= (uint32_t)f8 << (8 * i);
    }
    *reinterpret_cast<uint32_t*>(q + r * (int64_t)k + kb * 128 + lane * 4) = packed;
    if (lane == 0) scales[r * kblocks + kb] = scale;
  }
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" {

int b200_gemm_fp8(const b200_fp8_gemm_t* g, void* d, const void* a, const void* b, cudaStream_t stream) {
  if (g->m <= 0 || g->n <= 0) return 0;
  auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  if (g->k <= 0 || g->k % 16 != 0 || g->lda % 16 != 0 || g->ldb % 16 != 0 || !al(a) || !al(b)) return (int)cudaErrorNotSupported;
  if ((g->block_scale_a || g->block_scale_b) && g->k % 128 != 0) return (int)cudaErrorNotSupported;
  switch (g->out_dtype) {
    case B200_BF16: return launch_fp8<__nv_bfloat16>(g, d, a, b, stream);
    case B200_F16: return launch_fp8<__half>(g, d, a, b, stream);
    case B200_F32: return launch_fp8<float>(g, d, a, b, stream);
    default: return (int)cudaErrorNotSupported;
  }
}

int b200_quantize_fp8_1x128(int dtype, const void* x, void* q, float* scales, int64_t rows, int k, int64_t ldx, int e5m2,
                            cudaStream_t stream) {
  if (rows == 0 || k == 0) return 0;
  if (k % 128 != 0 || ldx % 4 != 0 || (reinterpret_cast<uintptr_t>(q) & 3)) return (int)cudaErrorNotSupported;
  const int64_t nblk = rows * (k / 128);
  const int grid = (int)std::min<int64_t>((nblk + 7) / 8, (int64_t)kSMs * 16);
  B200K_DISPATCH_FLOAT(dtype, T, (quant_1x128_kernel<T><<<grid, 256, 0, stream>>>((const T*)x, (uint8_t*)q, scales, rows, k, ldx, e5m2)));
  B200K_LAUNCH_RET();
}

}  // extern "C"
