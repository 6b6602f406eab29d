// Implicit-GEMM 2-D convolution on tcgen05 tensor cores: forward, data gradient and weight gradient for
// channels-last (NHWC) bf16/fp16 tensors, any filter size up to 7x7, stride 1 or 2, zero padding, groups 1.
//
// No im2col buffer exists anywhere.  The GEMM's K dimension runs over (filter tap, 64-channel chunk); for every
// such step TMA fetches a box [images x rows x columns x 64 channels] of the activation, shifted by the tap's
// offset, straight into the 128-byte-swizzled shared-memory layout the tensor core reads.  Pixels that fall
// into the padding are out of the tensor map's bounds and arrive as zeros.  A stride-2 convolution samples
// every other pixel: it reads through four tensor maps, one per (row, column) parity, whose strides skip the
// pixels in between, so the boxes stay dense.
//
//   forward  y[p, k]  = sum_{tap, c} x[p + tap, c] * w[k, tap, c]        A = x boxes (K-major), B = w (K-major)
//   dgrad    dx[p, c] = sum_{tap, k} dy[p' + tap', k] * w[k, tap, c]     A = dy boxes (K-major), B = w (MN-major),
//            one launch per stride-parity class of p, each with the taps that reach that class
//   wgrad    dw[k, tap, c] = sum_p dy[p, k] * x[p + tap, c]              A = dy boxes, B = x boxes (both MN-major),
//            K runs over pixels, split over CTAs, fp32 partial sums added with red.global
//
// One CTA owns a 128 x 128 accumulator tile in TMEM (two buffers, so the epilogue of a tile overlaps the
// main loop of the next one); warp 0 issues TMA, warp 1 issues tcgen05.mma, warps 2-5 drain TMEM.  The
// kernels are persistent over tiles with one CTA per SM.  Every mbarrier wait is bounded.
//
// Parity: reference torch_musa/csrc/aten/ops/Conv.cpp:129-155,379-461 (vendor-library forward / backward-data /
// backward-weight convolutions).
#include "attention_common.cuh"
#include "b200_kernels.h"

#include <algorithm>
#include <mutex>
#include <vector>

namespace b200k {
namespace convdev {
using namespace attndev;

constexpr int BM = 128, BN = 128, BK = 64;
constexpr int kStages = 6, kAccStages = 2, kTmemCols = 256;
constexpr int kATile = BM * BK * 2, kBTile = BN * BK * 2, kStageBytes = kATile + kBTile;
constexpr int kMaxTaps = 49;
constexpr int kThreads = 192;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment*/ + 256 /*barriers*/;

struct Tap {
  short dh, dw;  // offset of the tap in the (sub-sampled) pixel grid of the box operand
  short wrs;     // r * S + s: the tap's slab in the weight tensor
  short map;     // which parity map the box operand is read through
};

struct Maps {
  CUtensorMap box[4];  // pixel-box operand, one map per stride parity
  CUtensorMap other;   // weights (forward / dgrad) or dy (wgrad)
};

struct PixParams {
  int n_t, th, tw, rows;  // tile = n_t images x th rows x tw columns of output positions; rows = product <= 128
  int tiles_n, tiles_h, tiles_w, tiles_c;
  int N, Hg, Wg;  // extent of the output-position grid this launch covers
  int n_taps, k_chunks;
  int a_bytes;
  long long out_sn, out_sh, out_sw, out_off;  // element strides of the output for image / grid row / grid column
  int c_out;
  const void* bias;
  int relu;
  uint32_t idesc;
  int* status;
  Tap taps[kMaxTaps];
};

struct Smem {
  uint8_t* a;
  uint8_t* b;
  uint64_t *full, *empty, *tfull, *tempty;
  uint32_t* tmem_slot;
  volatile int* abort_flag;
};

__device__ __forceinline__ Smem carve(uint8_t* raw) {
  Smem s;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  s.a = base;
  s.b = base + kStages * kATile;
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + kStages * kStageBytes);
  s.full = bars;
  s.empty = bars + kStages;
  s.tfull = bars + 2 * kStages;
  s.tempty = bars + 2 * kStages + kAccStages;
  s.tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 2 * kAccStages);
  s.abort_flag = reinterpret_cast<volatile int*>(s.tmem_slot + 1);
  return s;
}

__device__ __forceinline__ void setup(const Smem& s, const Maps& maps, int warp) {
  if (threadIdx.x == 0) {
    *s.abort_flag = 0;
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&s.full[i], 1);
      mbar_init(&s.empty[i], 1);
    }
    for (int i = 0; i < kAccStages; ++i) {
      mbar_init(&s.tfull[i], 1);
      mbar_init(&s.tempty[i], 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&maps.box[0]);
    prefetch_tmap(&maps.other);
  }
  if (warp == 1) {
    tmem_alloc(s.tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
}

__device__ __forceinline__ void teardown(const Smem& s, uint32_t tmem_base, int warp, int* status) {
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *s.abort_flag && status) atomicExch(status, 1);
}

// MMA issue for one pipeline stage: four K=16 steps.
template <bool A_KMAJOR, bool B_KMAJOR>
__device__ __forceinline__ void issue_stage(uint32_t tmem_d, uint32_t sa, uint32_t sb, uint32_t idesc, bool first) {
#pragma unroll
  for (int kk = 0; kk < BK / 16; ++kk) {
    // K-major: 16 elements = 32 B inside the 128-byte swizzle row; SBO = 8 rows x 128 B.
    // MN-major: 16 k-rows of 128 B = 2048 B; LBO = next 64-wide MN box (8 KB), SBO = 8 k-rows.
    const uint64_t adesc = A_KMAJOR ? make_desc(sa + kk * 32, 16, 1024) : make_desc(sa + kk * 2048, 8192, 1024);
    const uint64_t bdesc = B_KMAJOR ? make_desc(sb + kk * 32, 16, 1024) : make_desc(sb + kk * 2048, 8192, 1024);
    umma_f16(tmem_d, adesc, bdesc, idesc, (first && kk == 0) ? 0u : 1u);
  }
}

// ------------------------------------------------------------------ forward / data gradient
template <bool B_KMAJOR, typename OutT>
__global__ void __launch_bounds__(kThreads, 1)
conv_pix_kernel(const __grid_constant__ Maps maps, const __grid_constant__ PixParams p, OutT* __restrict__ out) {
  extern __shared__ uint8_t smem_raw[];
  const Smem s = carve(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  setup(s, maps, warp);
  const uint32_t tmem_base = *s.tmem_slot;
  const int total_tiles = p.tiles_n * p.tiles_h * p.tiles_w * p.tiles_c;
  const int k_steps = p.n_taps * p.k_chunks;

  auto decode = [&](int tile, int& ct, int& n0, int& h0, int& w0) {
    ct = tile % p.tiles_c;
    int r = tile / p.tiles_c;
    w0 = (r % p.tiles_w) * p.tw;
    r /= p.tiles_w;
    h0 = (r % p.tiles_h) * p.th;
    n0 = (r / p.tiles_h) * p.n_t;
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int ct, n0, h0, w0;
        decode(tile, ct, n0, h0, w0);
        for (int ks = 0; ks < k_steps; ++ks) {
          const Tap tap = p.taps[ks / p.k_chunks];
          const int cc = ks % p.k_chunks;
          if (!mbar_wait(&s.empty[stage], phase ^ 1, s.abort_flag)) { ok = false; break; }
          mbar_expect_tx(&s.full[stage], (uint32_t)(p.a_bytes + kBTile));
          uint8_t* sa = s.a + stage * kATile;
          uint8_t* sb = s.b + stage * kBTile;
          tma_load_4d(sa, &maps.box[tap.map], &s.full[stage], cc * BK, w0 + tap.dw, h0 + tap.dh, n0);
          if constexpr (B_KMAJOR) {
            tma_load_3d(sb, &maps.other, &s.full[stage], cc * BK, tap.wrs, ct * BN);
          } else {
            tma_load_3d(sb, &maps.other, &s.full[stage], ct * BN, tap.wrs, cc * BK);
            tma_load_3d(sb + 8192, &maps.other, &s.full[stage], ct * BN + 64, tap.wrs, cc * BK);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(&s.tempty[acc], acc_phase ^ 1, s.abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int ks = 0; ks < k_steps; ++ks) {
          if (!mbar_wait(&s.full[stage], phase, s.abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_stage<true, B_KMAJOR>(tmem_d, smem_u32(s.a + stage * kATile), smem_u32(s.b + stage * kBTile), p.idesc,
                                      ks == 0);
          umma_commit(&s.empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&s.tfull[acc]);
        if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const int row = q * 32 + lane;
    const int per_img = p.th * p.tw;
    const int ni = row / per_img, rem = row - ni * per_img;
    const int ti = rem / p.tw, tj = rem - ti * p.tw;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      int ct, n0, h0, w0;
      decode(tile, ct, n0, h0, w0);
      if (!mbar_wait(&s.tfull[acc], acc_phase, s.abort_flag)) break;
      tc_fence_after();
      const bool valid = row < p.rows && n0 + ni < p.N && h0 + ti < p.Hg && w0 + tj < p.Wg;
      OutT* drow = out + p.out_off + (long long)(n0 + ni) * p.out_sn + (long long)(h0 + ti) * p.out_sh +
                   (long long)(w0 + tj) * p.out_sw + ct * BN;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = ct * BN + c * 32;
        if (col0 >= p.c_out) break;
        uint32_t raw[32];
        tmem_ld32(taddr + (uint32_t)(c * 32), raw);
        tmem_ld_wait();
        if (valid) {
          const int nvalid = min(32, p.c_out - col0);
          float v[32];
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __uint_as_float(raw[e]);
          if (p.bias) {
            const OutT* bp = reinterpret_cast<const OutT*>(p.bias) + col0;
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (e < nvalid) v[e] += ToF<OutT>::to(bp[e]);
          }
          if (p.relu) {
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = fmaxf(v[e], 0.f);
          }
          store_chunk<OutT>(drow + c * 32, v, nvalid, true);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.tempty[acc]);
      if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
    }
  }
  teardown(s, tmem_base, warp, p.status);
}

// ------------------------------------------------------------------ weight gradient
struct WgradParams {
  int n_t, th, tw;  // pixel rectangle of one K step: exactly 64 positions
  int tiles_n, tiles_h, tiles_w;
  int tiles_m, tiles_nc;  // output tiles: Cout / 128 and channel tiles per tap
  int n_taps, splits, steps_per_split;
  int c_out, c_in, rs;  // dw is [c_out][rs][c_in] fp32
  uint32_t idesc;
  int* status;
  Tap taps[kMaxTaps];
};

__global__ void __launch_bounds__(kThreads, 1)
conv_wgrad_kernel(const __grid_constant__ Maps maps, const __grid_constant__ WgradParams p, float* __restrict__ dw) {
  extern __shared__ uint8_t smem_raw[];
  const Smem s = carve(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  setup(s, maps, warp);
  const uint32_t tmem_base = *s.tmem_slot;
  const int out_tiles = p.tiles_m * p.n_taps * p.tiles_nc;
  const int total_tiles = out_tiles * p.splits;
  const int pix_tiles = p.tiles_n * p.tiles_h * p.tiles_w;

  auto decode = [&](int tile, int& mt, int& tap_i, int& nc, int& s0, int& s1) {
    const int split = tile / out_tiles;
    int r = tile - split * out_tiles;
    mt = r % p.tiles_m;
    r /= p.tiles_m;
    nc = r % p.tiles_nc;
    tap_i = r / p.tiles_nc;
    s0 = split * p.steps_per_split;
    s1 = min(pix_tiles, s0 + p.steps_per_split);
  };

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int mt, tap_i, nc, s0, s1;
        decode(tile, mt, tap_i, nc, s0, s1);
        const Tap tap = p.taps[tap_i];
        for (int st = s0; st < s1; ++st) {
          int r = st;
          const int w0 = (r % p.tiles_w) * p.tw;
          r /= p.tiles_w;
          const int h0 = (r % p.tiles_h) * p.th;
          const int n0 = (r / p.tiles_h) * p.n_t;
          if (!mbar_wait(&s.empty[stage], phase ^ 1, s.abort_flag)) { ok = false; break; }
          mbar_expect_tx(&s.full[stage], (uint32_t)kStageBytes);
          uint8_t* sa = s.a + stage * kATile;
          uint8_t* sb = s.b + stage * kBTile;
          // A = dy: rows are the 64 pixels (K), 128 output channels (M) in two 64-wide boxes
          tma_load_4d(sa, &maps.other, &s.full[stage], mt * BM, w0, h0, n0);
          tma_load_4d(sa + 8192, &maps.other, &s.full[stage], mt * BM + 64, w0, h0, n0);
          // B = x shifted by the tap: 64 pixels (K) x 128 input channels (N)
          tma_load_4d(sb, &maps.box[tap.map], &s.full[stage], nc * BN, w0 + tap.dw, h0 + tap.dh, n0);
          tma_load_4d(sb + 8192, &maps.box[tap.map], &s.full[stage], nc * BN + 64, w0 + tap.dw, h0 + tap.dh, n0);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        int mt, tap_i, nc, s0, s1;
        decode(tile, mt, tap_i, nc, s0, s1);
        if (!mbar_wait(&s.tempty[acc], acc_phase ^ 1, s.abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int st = s0; st < s1; ++st) {
          if (!mbar_wait(&s.full[stage], phase, s.abort_flag)) { ok = false; break; }
          tc_fence_after();
          issue_stage<false, false>(tmem_d, smem_u32(s.a + stage * kATile), smem_u32(s.b + stage * kBTile), p.idesc,
                                    st == s0);
          umma_commit(&s.empty[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(&s.tfull[acc]);
        if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
      }
    }
    __syncwarp();
  } else {
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const int row = q * 32 + lane;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x) {
      int mt, tap_i, nc, s0, s1;
      decode(tile, mt, tap_i, nc, s0, s1);
      if (!mbar_wait(&s.tfull[acc], acc_phase, s.abort_flag)) break;
      tc_fence_after();
      const int k = mt * BM + row;
      float* drow = dw + ((long long)k * p.rs + p.taps[tap_i].wrs) * p.c_in + nc * BN;
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = nc * BN + c * 32;
        if (col0 >= p.c_in) break;
        uint32_t raw[32];
        tmem_ld32(taddr + (uint32_t)(c * 32), raw);
        tmem_ld_wait();
        if (k < p.c_out && s1 > s0) {
          const int nvalid = min(32, p.c_in - col0);
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (e < nvalid) atomicAdd(drow + c * 32 + e, __uint_as_float(raw[e]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s.tempty[acc]);
      if (++acc == kAccStages) { acc = 0; acc_phase ^= 1; }
    }
  }
  teardown(s, tmem_base, warp, p.status);
}

// ------------------------------------------------------------------ host side
EncodeTiledFn encoder() {
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
  return enc;
}

CUtensorMapDataType map_dtype(int dtype) {
  return dtype == B200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
}

// NHWC activation [N, H, W, C] sampled at rows hp, hp + sh, ... and columns wp, wp + sw, ...
bool make_pixel_map(CUtensorMap* out, const void* base, int dtype, int64_t N, int64_t H, int64_t W, int64_t C, int sh,
                    int sw, int hp, int wp, int box_c, int tw, int th, int n_t) {
  EncodeTiledFn enc = encoder();
  if (!enc) return false;
  const int64_t Hs = (H - hp + sh - 1) / sh, Ws = (W - wp + sw - 1) / sw;
  if (Hs <= 0 || Ws <= 0) return false;
  const char* p = static_cast<const char*>(base) + ((int64_t)hp * W + wp) * C * 2;
  cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)Ws, (cuuint64_t)Hs, (cuuint64_t)N};
  cuuint64_t strides[3] = {(cuuint64_t)(sw * C * 2), (cuuint64_t)(sh * W * C * 2), (cuuint64_t)(H * W * C * 2)};
  cuuint32_t box[4] = {(cuuint32_t)box_c, (cuuint32_t)tw, (cuuint32_t)th, (cuuint32_t)n_t};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return enc(out, map_dtype(dtype), 4, const_cast<char*>(p), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Weights [K][R*S][C] (channels-last filter): box {64 channels, 1 tap, rows filters}
bool make_weight_map(CUtensorMap* out, const void* base, int dtype, int64_t K, int64_t RS, int64_t C, int rows) {
  EncodeTiledFn enc = encoder();
  if (!enc) return false;
  cuuint64_t dims[3] = {(cuuint64_t)C, (cuuint64_t)RS, (cuuint64_t)K};
  cuuint64_t strides[2] = {(cuuint64_t)(C * 2), (cuuint64_t)(RS * C * 2)};
  cuuint32_t box[3] = {64, 1, (cuuint32_t)rows};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(out, map_dtype(dtype), 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int floor_div(int a, int b) { return a >= 0 ? a / b : -((-a + b - 1) / b); }
int pos_mod(int a, int b) { return ((a % b) + b) % b; }

// Rectangle (n_t, th, tw) of output positions with n_t * th * tw <= limit (== limit when `exact`) that wastes the
// fewest tile rows over an N x H x W grid.
void pick_rect(int64_t N, int H, int W, int limit, bool exact, int& n_t, int& th, int& tw) {
  double best = -1;
  n_t = 1, th = 1, tw = 1;
  for (int w = 1; w <= std::min(limit, 256); ++w) {
    for (int h = 1; h * w <= limit && h <= 256; ++h) {
      int nmax = limit / (h * w);
      for (int n = 1; n <= std::min(nmax, 256); n = (n < 4 ? n + 1 : n * 2)) {
        if (exact && n * h * w != limit) continue;
        if (w > W + 8 || h > H + 8) continue;
        const double tiles = (double)((N + n - 1) / n) * ((H + h - 1) / h) * ((W + w - 1) / w);
        const double eff = (double)N * H * W / (tiles * limit);
        // prefer wide boxes at equal efficiency: fewer, longer TMA rows
        const double score = eff + 1e-4 * w + 1e-6 * h;
        if (score > best) { best = score; n_t = n; th = h; tw = w; }
      }
    }
  }
}

int* status_word() {
  static int* w = [] {
    int* p = nullptr;
    if (cudaHostAlloc((void**)&p, sizeof(int), cudaHostAllocMapped) != cudaSuccess) {
      (void)cudaGetLastError();
      return (int*)nullptr;
    }
    *p = 0;
    return p;
  }();
  return w;
}
int* device_status() {
  int* h = status_word();
  int* d = nullptr;
  if (!h || cudaHostGetDevicePointer((void**)&d, h, 0) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  return d;
}

int sm_count() {
  static int n = [] {
    int dev = 0, v = 148;
    cudaGetDevice(&dev);
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) (void)cudaGetLastError();
    return v;
  }();
  return n;
}

template <typename K>
bool opt_in_smem(K kernel) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) == cudaSuccess;
}

uint32_t make_idesc(int dtype, bool a_kmajor, bool b_kmajor) {
  const uint32_t fmt = dtype == B200_BF16 ? 1u : 0u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_kmajor ? 0u : 1u) << 15) | ((b_kmajor ? 0u : 1u) << 16) |
         ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

bool supported(const b200_conv_t* d) {
  if (!encoder()) return false;
  if (d->dtype != B200_BF16 && d->dtype != B200_F16) return false;
  if (d->sh < 1 || d->sh > 2 || d->sw < 1 || d->sw > 2) return false;
  if (d->R < 1 || d->S < 1 || d->R * d->S > kMaxTaps) return false;
  if (d->C % 8 != 0 || d->K % 8 != 0) return false;  // 16-byte rows for TMA and the vector stores
  if (d->N < 1 || d->Ho < 1 || d->Wo < 1) return false;
  if (d->ph < 0 || d->pw < 0 || d->ph >= 32 || d->pw >= 32) return false;
  return true;
}

template <bool B_KMAJOR>
int launch_pix(const Maps& maps, const PixParams& p, int dtype, void* out, cudaStream_t stream) {
  const int total = p.tiles_n * p.tiles_h * p.tiles_w * p.tiles_c;
  const int grid = std::min(total, sm_count());
  if (dtype == B200_BF16) {
    auto k = conv_pix_kernel<B_KMAJOR, __nv_bfloat16>;
    if (!opt_in_smem(k)) return (int)cudaGetLastError();
    k<<<grid, kThreads, kSmemBytes, stream>>>(maps, p, static_cast<__nv_bfloat16*>(out));
  } else {
    auto k = conv_pix_kernel<B_KMAJOR, __half>;
    if (!opt_in_smem(k)) return (int)cudaGetLastError();
    k<<<grid, kThreads, kSmemBytes, stream>>>(maps, p, static_cast<__half*>(out));
  }
  return (int)cudaGetLastError();
}

}  // namespace convdev
}  // namespace b200k

using namespace b200k::convdev;

extern "C" int b200_conv_supported(const b200_conv_t* d) { return supported(d) ? 1 : 0; }

extern "C" int b200_conv_status(int clear) {
  int* w = status_word();
  if (!w) return 0;
  int v = *w;
  if (clear) *w = 0;
  return v;
}

extern "C" int b200_conv_fwd(const b200_conv_t* d, void* y, const void* x, const void* w, const void* bias, int relu,
                             cudaStream_t stream) {
  if (!supported(d)) return (int)cudaErrorNotSupported;
  Maps maps{};
  PixParams p{};
  int n_t, th, tw;
  pick_rect(d->N, (int)d->Ho, (int)d->Wo, BM, false, n_t, th, tw);
  p.n_t = n_t, p.th = th, p.tw = tw, p.rows = n_t * th * tw;
  p.tiles_n = (int)((d->N + n_t - 1) / n_t);
  p.tiles_h = (int)((d->Ho + th - 1) / th);
  p.tiles_w = (int)((d->Wo + tw - 1) / tw);
  p.tiles_c = (int)((d->K + BN - 1) / BN);
  p.N = (int)d->N, p.Hg = (int)d->Ho, p.Wg = (int)d->Wo;
  p.k_chunks = (int)((d->C + BK - 1) / BK);
  p.a_bytes = p.rows * BK * 2;
  p.out_sn = d->Ho * d->Wo * d->K, p.out_sh = d->Wo * d->K, p.out_sw = d->K, p.out_off = 0;
  p.c_out = (int)d->K;
  p.bias = bias, p.relu = relu;
  p.idesc = make_idesc(d->dtype, true, true);
  p.status = device_status();
  bool have[4] = {false, false, false, false};
  for (int r = 0; r < d->R; ++r)
    for (int s = 0; s < d->S; ++s) {
      Tap t;
      const int hp = pos_mod(r - d->ph, d->sh), wp = pos_mod(s - d->pw, d->sw);
      t.map = (short)(hp * d->sw + wp);
      t.dh = (short)floor_div(r - d->ph, d->sh);
      t.dw = (short)floor_div(s - d->pw, d->sw);
      t.wrs = (short)(r * d->S + s);
      if (hp >= d->H || wp >= d->W) continue;  // this parity has no pixel at all
      if (!have[t.map]) {
        if (!make_pixel_map(&maps.box[t.map], x, d->dtype, d->N, d->H, d->W, d->C, d->sh, d->sw, hp, wp, BK, tw, th, n_t))
          return (int)cudaErrorInvalidValue;
        have[t.map] = true;
      }
      p.taps[p.n_taps++] = t;
    }
  if (p.n_taps == 0) return (int)cudaErrorInvalidValue;
  if (!have[0]) maps.box[0] = maps.box[p.taps[0].map];  // only prefetched
  if (!make_weight_map(&maps.other, w, d->dtype, d->K, d->R * d->S, d->C, BN)) return (int)cudaErrorInvalidValue;
  return launch_pix<true>(maps, p, d->dtype, y, stream);
}

extern "C" int b200_conv_dgrad(const b200_conv_t* d, void* dx, const void* dy, const void* w, cudaStream_t stream) {
  if (!supported(d)) return (int)cudaErrorNotSupported;
  // one launch per parity class (a, b) of the input position; classes no tap reaches stay zero
  bool any_empty = false;
  struct Launch { Maps maps; PixParams p; };
  std::vector<Launch> launches;
  for (int a = 0; a < d->sh; ++a)
    for (int b = 0; b < d->sw; ++b) {
      const int Hg = (int)((d->H - a + d->sh - 1) / d->sh), Wg = (int)((d->W - b + d->sw - 1) / d->sw);
      if (Hg <= 0 || Wg <= 0) continue;
      Launch L{};
      PixParams& p = L.p;
      for (int r = 0; r < d->R; ++r) {
        if (pos_mod(a + d->ph - r, d->sh) != 0) continue;
        for (int s = 0; s < d->S; ++s) {
          if (pos_mod(b + d->pw - s, d->sw) != 0) continue;
          Tap t;
          t.map = 0;
          t.dh = (short)floor_div(a + d->ph - r, d->sh);
          t.dw = (short)floor_div(b + d->pw - s, d->sw);
          t.wrs = (short)(r * d->S + s);
          p.taps[p.n_taps++] = t;
        }
      }
      if (p.n_taps == 0) { any_empty = true; continue; }
      int n_t, th, tw;
      pick_rect(d->N, Hg, Wg, BM, false, n_t, th, tw);
      p.n_t = n_t, p.th = th, p.tw = tw, p.rows = n_t * th * tw;
      p.tiles_n = (int)((d->N + n_t - 1) / n_t);
      p.tiles_h = (Hg + th - 1) / th;
      p.tiles_w = (Wg + tw - 1) / tw;
      p.tiles_c = (int)((d->C + BN - 1) / BN);
      p.N = (int)d->N, p.Hg = Hg, p.Wg = Wg;
      p.k_chunks = (int)((d->K + BK - 1) / BK);
      p.a_bytes = p.rows * BK * 2;
      p.out_sn = d->H * d->W * d->C, p.out_sh = (long long)d->sh * d->W * d->C, p.out_sw = (long long)d->sw * d->C;
      p.out_off = ((long long)a * d->W + b) * d->C;
      p.c_out = (int)d->C;
      p.idesc = make_idesc(d->dtype, true, false);
      p.status = device_status();
      if (!make_pixel_map(&L.maps.box[0], dy, d->dtype, d->N, d->Ho, d->Wo, d->K, 1, 1, 0, 0, BK, tw, th, n_t))
        return (int)cudaErrorInvalidValue;
      if (!make_weight_map(&L.maps.other, w, d->dtype, d->K, d->R * d->S, d->C, 64)) return (int)cudaErrorInvalidValue;
      launches.push_back(L);
    }
  if (any_empty) {
    cudaError_t e = cudaMemsetAsync(dx, 0, (size_t)d->N * d->H * d->W * d->C * 2, stream);
    if (e != cudaSuccess) return (int)e;
  }
  for (auto& L : launches) {
    int e = launch_pix<false>(L.maps, L.p, d->dtype, dx, stream);
    if (e != 0) return e;
  }
  return 0;
}

namespace b200k { namespace convdev { bool g_wgrad_deterministic = false; } }
// With `on`, every output tile of the weight gradient is produced by ONE CTA in a fixed pixel order (no split over
// pixels, so no fp32 atomics whose order varies from run to run): slower, bit-reproducible.
extern "C" void b200_conv_set_deterministic(int on) { g_wgrad_deterministic = on != 0; }

extern "C" int b200_conv_wgrad(const b200_conv_t* d, float* dw_f32, const void* dy, const void* x,
                               cudaStream_t stream) {
  if (!supported(d)) return (int)cudaErrorNotSupported;
  Maps maps{};
  WgradParams p{};
  int n_t, th, tw;
  pick_rect(d->N, (int)d->Ho, (int)d->Wo, BK, true, n_t, th, tw);
  p.n_t = n_t, p.th = th, p.tw = tw;
  p.tiles_n = (int)((d->N + n_t - 1) / n_t);
  p.tiles_h = (int)((d->Ho + th - 1) / th);
  p.tiles_w = (int)((d->Wo + tw - 1) / tw);
  p.tiles_m = (int)((d->K + BM - 1) / BM);
  p.tiles_nc = (int)((d->C + BN - 1) / BN);
  p.c_out = (int)d->K, p.c_in = (int)d->C, p.rs = d->R * d->S;
  p.idesc = make_idesc(d->dtype, false, false);
  p.status = device_status();
  bool have[4] = {false, false, false, false};
  for (int r = 0; r < d->R; ++r)
    for (int s = 0; s < d->S; ++s) {
      Tap t;
      const int hp = pos_mod(r - d->ph, d->sh), wp = pos_mod(s - d->pw, d->sw);
      t.map = (short)(hp * d->sw + wp);
      t.dh = (short)floor_div(r - d->ph, d->sh);
      t.dw = (short)floor_div(s - d->pw, d->sw);
      t.wrs = (short)(r * d->S + s);
      if (hp >= d->H || wp >= d->W) continue;
      if (!have[t.map]) {
        if (!make_pixel_map(&maps.box[t.map], x, d->dtype, d->N, d->H, d->W, d->C, d->sh, d->sw, hp, wp, 64, tw, th, n_t))
          return (int)cudaErrorInvalidValue;
        have[t.map] = true;
      }
      p.taps[p.n_taps++] = t;
    }
  if (p.n_taps == 0) return 0;
  if (!have[0]) maps.box[0] = maps.box[p.taps[0].map];
  if (!make_pixel_map(&maps.other, dy, d->dtype, d->N, d->Ho, d->Wo, d->K, 1, 1, 0, 0, 64, tw, th, n_t))
    return (int)cudaErrorInvalidValue;
  const int out_tiles = p.tiles_m * p.n_taps * p.tiles_nc;
  const int pix_tiles = p.tiles_n * p.tiles_h * p.tiles_w;
  int splits = g_wgrad_deterministic ? 1 : std::max(1, (2 * sm_count() + out_tiles - 1) / out_tiles);
  splits = std::min(splits, pix_tiles);
  p.steps_per_split = (pix_tiles + splits - 1) / splits;
  p.splits = (pix_tiles + p.steps_per_split - 1) / p.steps_per_split;
  const int grid = std::min(out_tiles * p.splits, sm_count());
  if (!opt_in_smem(conv_wgrad_kernel)) return (int)cudaGetLastError();
  conv_wgrad_kernel<<<grid, kThreads, kSmemBytes, stream>>>(maps, p, dw_f32);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------ few-channel ("stem") convolutions
// With C <= 8 input channels a tap holds 16 bytes per pixel and the generic path would spend a whole 128-byte
// K step on it.  Here the caller provides the image physically zero-padded to [N, Hp, Wp, 8] (Hp = H + 2 ph,
// Wp = W + 2 pw) and one K step covers a whole filter ROW: the S taps x 8 channels of one output pixel are
// S * 8 <= 64 consecutive elements of that layout.  Consecutive output pixels start sw * 8 elements apart,
// which is less than the 64 elements a row of the box spans, so output columns are processed in `cls_n`
// interleaved classes (wo = cls_n * j + cls) whose starts are >= 64 elements apart: within a class the rows of
// a box do not overlap and an ordinary tiled tensor map describes them.  Filters are packed as [K][R][64].
namespace b200k {
namespace convdev {

struct StemGeom {
  int cls_n;        // number of output-column classes
  int64_t Hp, Wp;   // padded image extent
};

bool stem_geom(const b200_conv_t* d, StemGeom* g) {
  if (d->dtype != B200_BF16 && d->dtype != B200_F16) return false;
  if (d->C != 8 || d->S * 8 > 64 || d->R > kMaxTaps || d->K % 8 != 0) return false;
  if (d->sh < 1 || d->sh > 2 || d->sw < 1 || d->sw > 2) return false;
  g->cls_n = (64 + d->sw * 8 - 1) / (d->sw * 8);  // smallest class count with starts >= 64 elements apart
  g->Hp = d->H + 2 * d->ph;
  g->Wp = d->W + 2 * d->pw;
  // the last pixel's row of 64 elements must end inside its image row
  if ((d->Wo - 1) * d->sw + 8 > g->Wp) return false;
  return encoder() != nullptr;
}

// Rows of 64 elements of the padded image: row (n, h2, j) starts at pixel (hp + sh * h2, (cls + cls_n * j) * sw).
bool make_stem_map(CUtensorMap* out, const void* xpad, const b200_conv_t* d, const StemGeom& g, int hp, int cls, int tw,
                   int th, int n_t) {
  const int64_t Wc = (d->Wo - cls + g.cls_n - 1) / g.cls_n;
  const int64_t Hs = (g.Hp - hp + d->sh - 1) / d->sh;
  if (Wc <= 0 || Hs <= 0) return false;
  const char* p = static_cast<const char*>(xpad) + ((int64_t)hp * g.Wp + (int64_t)cls * d->sw) * 8 * 2;
  cuuint64_t dims[4] = {64, (cuuint64_t)Wc, (cuuint64_t)Hs, (cuuint64_t)d->N};
  cuuint64_t strides[3] = {(cuuint64_t)(g.cls_n * d->sw * 8 * 2), (cuuint64_t)(d->sh * g.Wp * 8 * 2),
                           (cuuint64_t)(g.Hp * g.Wp * 8 * 2)};
  cuuint32_t box[4] = {64, (cuuint32_t)tw, (cuuint32_t)th, (cuuint32_t)n_t};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  return encoder()(out, map_dtype(d->dtype), 4, const_cast<char*>(p), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace convdev
}  // namespace b200k

extern "C" int b200_conv_stem_supported(const b200_conv_t* d) {
  StemGeom g;
  return stem_geom(d, &g) ? 1 : 0;
}

// y[N, Ho, Wo, K] from xpad[N, Hp, Wp, 8] and wpack[K][R][64] (element s * 8 + c of a row; the tail is zero).
extern "C" int b200_conv_stem_fwd(const b200_conv_t* d, void* y, const void* xpad, const void* wpack, const void* bias,
                                  int relu, cudaStream_t stream) {
  StemGeom g;
  if (!stem_geom(d, &g)) return (int)cudaErrorNotSupported;
  for (int cls = 0; cls < g.cls_n; ++cls) {
    const int Wc = (int)((d->Wo - cls + g.cls_n - 1) / g.cls_n);
    if (Wc <= 0) continue;
    Maps maps{};
    PixParams p{};
    int n_t, th, tw;
    pick_rect(d->N, (int)d->Ho, Wc, BM, false, n_t, th, tw);
    p.n_t = n_t, p.th = th, p.tw = tw, p.rows = n_t * th * tw;
    p.tiles_n = (int)((d->N + n_t - 1) / n_t);
    p.tiles_h = (int)((d->Ho + th - 1) / th);
    p.tiles_w = (Wc + tw - 1) / tw;
    p.tiles_c = (int)((d->K + BN - 1) / BN);
    p.N = (int)d->N, p.Hg = (int)d->Ho, p.Wg = Wc;
    p.k_chunks = 1;
    p.a_bytes = p.rows * BK * 2;
    p.out_sn = d->Ho * d->Wo * d->K, p.out_sh = d->Wo * d->K, p.out_sw = (long long)g.cls_n * d->K;
    p.out_off = (long long)cls * d->K;
    p.c_out = (int)d->K;
    p.bias = bias, p.relu = relu;
    p.idesc = make_idesc(d->dtype, true, true);
    p.status = device_status();
    bool have[2] = {false, false};
    for (int r = 0; r < d->R; ++r) {
      const int hp = r % d->sh;
      if (!have[hp]) {
        if (!make_stem_map(&maps.box[hp], xpad, d, g, hp, cls, tw, th, n_t)) return (int)cudaErrorInvalidValue;
        have[hp] = true;
      }
      Tap t;
      t.map = (short)hp, t.dh = (short)(r / d->sh), t.dw = 0, t.wrs = (short)r;
      p.taps[p.n_taps++] = t;
    }
    if (!make_weight_map(&maps.other, wpack, d->dtype, d->K, d->R, 64, BN)) return (int)cudaErrorInvalidValue;
    int e = launch_pix<true>(maps, p, d->dtype, y, stream);
    if (e != 0) return e;
  }
  return 0;
}

// dwpack_f32[K][R][64] += sum over pixels of dy[N, Ho, Wo, K] x rows of xpad (fp32, zeroed by the caller).
extern "C" int b200_conv_stem_wgrad(const b200_conv_t* d, float* dwpack_f32, const void* dy, const void* xpad,
                                    cudaStream_t stream) {
  StemGeom g;
  if (!stem_geom(d, &g)) return (int)cudaErrorNotSupported;
  if (!opt_in_smem(conv_wgrad_kernel)) return (int)cudaGetLastError();
  for (int cls = 0; cls < g.cls_n; ++cls) {
    const int Wc = (int)((d->Wo - cls + g.cls_n - 1) / g.cls_n);
    if (Wc <= 0) continue;
    Maps maps{};
    WgradParams p{};
    int n_t, th, tw;
    pick_rect(d->N, (int)d->Ho, Wc, BK, true, n_t, th, tw);
    p.n_t = n_t, p.th = th, p.tw = tw;
    p.tiles_n = (int)((d->N + n_t - 1) / n_t);
    p.tiles_h = (int)((d->Ho + th - 1) / th);
    p.tiles_w = (Wc + tw - 1) / tw;
    p.tiles_m = (int)((d->K + BM - 1) / BM);
    p.tiles_nc = 1;
    p.c_out = (int)d->K, p.c_in = 64, p.rs = d->R;
    p.idesc = make_idesc(d->dtype, false, false);
    p.status = device_status();
    bool have[2] = {false, false};
    for (int r = 0; r < d->R; ++r) {
      const int hp = r % d->sh;
      if (!have[hp]) {
        if (!make_stem_map(&maps.box[hp], xpad, d, g, hp, cls, tw, th, n_t)) return (int)cudaErrorInvalidValue;
        have[hp] = true;
      }
      Tap t;
      t.map = (short)hp, t.dh = (short)(r / d->sh), t.dw = 0, t.wrs = (short)r;
      p.taps[p.n_taps++] = t;
    }
    // dy of this class: columns cls, cls + cls_n, ...
    if (!make_pixel_map(&maps.other, dy, d->dtype, d->N, d->Ho, d->Wo, d->K, 1, g.cls_n, 0, cls, 64, tw, th, n_t))
      return (int)cudaErrorInvalidValue;
    const int out_tiles = p.tiles_m * p.n_taps;
    const int pix_tiles = p.tiles_n * p.tiles_h * p.tiles_w;
    int splits = std::max(1, (2 * sm_count() + out_tiles - 1) / out_tiles);
    splits = std::min(splits, pix_tiles);
    p.steps_per_split = (pix_tiles + splits - 1) / splits;
    p.splits = (pix_tiles + p.steps_per_split - 1) / p.steps_per_split;
    const int grid = std::min(out_tiles * p.splits, sm_count());
    conv_wgrad_kernel<<<grid, kThreads, kSmemBytes, stream>>>(maps, p, dwpack_f32);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}
