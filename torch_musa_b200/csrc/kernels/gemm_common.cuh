// Device-side building blocks shared by the tcgen05 GEMM kernels: mbarrier / TMA / TMEM / tcgen05 PTX
// wrappers, shared-memory matrix descriptors, the epilogue helpers and the parameter block.
#pragma once

#include "common.cuh"

#include <cuda.h>

#include <cstdlib>

namespace b200k {
namespace gemmdev {

constexpr long long kWaitCycles = 4000000000ll;  // ~2 s: far beyond any legitimate wait inside one GPU
// Limit that the pipeline waits of this translation unit use.  Kernels that also wait for other ranks raise it
// to the process group's limit before they launch (one copy per translation unit and device).
static __constant__ long long c_wait_cycles = kWaitCycles;

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait. Returns false when the wait gave up (abort flag set by anyone, or time-out).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try(bar, parity)) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (!mbar_try(bar, parity)) {
    if ((++spins & 0x3ff) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > c_wait_cycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// fp32 operands read as tf32 (the tensor core ignores the low 13 mantissa bits); K = 8 per instruction
__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100 format): 128-byte swizzle, version 1.
//   bits [0,14)  start address >> 4      bits [16,30) leading byte offset >> 4
//   bits [32,46) stride byte offset >> 4 bits [46,48) version = 1   bits [61,64) layout = 2 (SWIZZLE_128B)
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

struct Params {
  int m, n, k;
  int batch;
  int tiles_m, tiles_n;
  int64_t ldd;       // elements
  int64_t stride_d;  // elements between batches
  const void* bias;
  int bias_f32;
  int act;
  int accumulate;
  float alpha;
  uint32_t idesc;
  int* status;  // device word: set to 1 when a bounded wait expired
  // split-K: tile index = split * (tiles * batch) + tile; split s covers k-blocks [s * kb_per_split, ...) and
  // writes its partial product at d + s * split_stride
  int splits;
  int kb_per_split;
  int64_t split_stride;
  int group_m;   // row tiles per L2 group (see decode_tile)
};

// Row tiles per L2 group (see decode_tile).  Measured on the Llama-7B shapes (us, 74 SM pairs):
//   * both operands MN-major (weight gradients): one group over all row tiles re-reads the operands from DRAM
//     several times (1.06 GB against 134 MB of algorithmic bytes at 4096 x 12288 x 4096; L2 hit rate 57 % against
//     85 % for the K-major layout): groups of 4 row tiles bring 302 -> 265 at that shape, 110 -> 102 at 4096^3;
//   * K-major: while A (M x K x 2 bytes) is at most 64 MB one group covers every row tile (A stays resident, B
//     streams once); beyond that (K = 11008) groups of about 24 MB of A rows: 303 -> 291.
inline int gemm_group_m(int tile_rows, int m, int k, bool both_mn_major = false) {
  static const int forced = [] {   // experiment knob
    const char* e = std::getenv("B200_GEMM_GROUP_M");
    return e ? std::atoi(e) : 0;
  }();
  if (forced > 0) return forced;
  const long long per_tile = (long long)tile_rows * k * 2;
  const int tiles_m = (m + tile_rows - 1) / tile_rows;
  int g;
  if ((long long)m * k * 2 <= (64ll << 20)) {
    g = tiles_m > 0 ? tiles_m : 1;
  } else {
    long long q = (24ll << 20) / (per_tile > 0 ? per_tile : 1);
    g = (int)(q < 2 ? 2 : (q > 32 ? 32 : q));
  }
  if (both_mn_major && g > 4) g = 4;
  return g;
}




// Tile order inside one batch / split: groups of `group_m` row tiles are walked completely (row tile fastest, then
// the next column tile) before the next group starts.  The rows of A that a group touches (group_m x tile rows x K)
// then stay in L2 while every column tile streams past, instead of all of A being re-read from HBM once per column
// tile as soon as M x K outgrows the L2 (M = 16384, K = 4096 bf16 is 134 MB against 126 MB of L2).
__device__ __forceinline__ void decode_tile(int r, int tiles_m, int tiles_n, int group_m, int& mt, int& nt) {
  const int per_group = group_m * tiles_n;
  const int g = r / per_group;
  const int first = g * group_m;
  const int gsize = min(group_m, tiles_m - first);
  const int in_g = r - g * per_group;
  nt = in_g / gsize;
  mt = first + (in_g - nt * gsize);
}

__device__ __forceinline__ float apply_act(float v, int act) {
  switch (act) {
    case 1: return v > 0.f ? v : 0.f;
    case 2: return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
    case 3: return v / (1.f + __expf(-v));
    default: return v;
  }
}

template <typename OutT>
__device__ __forceinline__ void store_chunk(OutT* __restrict__ drow, const float (&v)[32], int ncols_valid, bool vec_ok) {
  if (vec_ok && ncols_valid == 32) {
    if constexpr (sizeof(OutT) == 2) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        Vec16<OutT> o;
#pragma unroll
        for (int e = 0; e < 8; ++e) o.v[e] = ToF<OutT>::from(v[q * 8 + e]);
        st16(drow + q * 8, o);
      }
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<float4*>(reinterpret_cast<float*>(drow) + q * 4) =
            make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
    }
  } else {
#pragma unroll
    for (int e = 0; e < 32; ++e)
      if (e < ncols_valid) drow[e] = ToF<OutT>::from(v[e]);
  }
}


}  // namespace gemmdev

// all-gather -> GEMM: the A operand [M, K] is assembled in local memory from the ranks' row shards by a few
// copier CTAs of the same launch while the other clusters already multiply the panels that have arrived.
struct AgParams {
  int enabled;
  int world, rank;
  int copier_pairs;          // clusters (from pair index 0) that copy instead of multiplying
  int panels_per_shard;      // 256-row panels in one rank's shard
  int64_t panel_bytes;       // 256 * K * 2
  const void* src[16];       // every rank's shard (peer-mapped; src[rank] is the local one)
  void* dst;                 // local [M, K]
  uint32_t* flags;           // local, one word per panel: epoch of the last call that completed it
  uint32_t* sig[16];         // signal pads (peer-mapped), slot [copier CTA][source rank]
  uint32_t epoch;            // this call: epoch = shards ready, epoch + 1 = peer finished pulling
  long long wait_cycles;     // limit of the waits on other ranks
};

// GEMM -> reduce-scatter: every rank multiplies into a partial [M, N] buffer of its arena, visiting the row panels
// of the other ranks first; per finished tile it raises a flag in the panel owner's arena.  A few reducer CTAs of
// the same launch wait for the flags of their own panels from every source rank, pull the partial panels with bulk
// copies into shared memory, sum them in fp32 and write this rank's [M / world, N] output rows.
struct RsParams {
  int enabled;
  int world, rank;
  int reducer_pairs;         // clusters (from pair index 0) that reduce instead of multiplying
  int panels_per_shard;
  int64_t panel_bytes;       // 256 * N * 2
  const void* src[16];       // every rank's partial buffer (peer-mapped)
  uint32_t* flag[16];        // every rank's flag table (peer-mapped): [source rank][panel in shard][n tile][cta of pair]
  uint32_t* sig[16];         // signal pads for the trailing barrier
  void* out;                 // local [M / world, N]
  uint32_t epoch;
  long long wait_cycles;     // limit of the waits on other ranks
};

// What the host decided for one problem: how many K-splits and which kernel family.
struct GemmPlan {
  int pair;          // 1: SM-pair kernel (256-row tiles), 0: single-CTA kernel (128-row tiles)
  int dynamic;       // pair kernel: cluster-launch-control schedule
  int splits;        // 1 = no split-K
  int kb_per_split;
};

// host helpers implemented in gemm_tcgen05.cu
bool gemm_make_map(CUtensorMap* out, const void* ptr, int dtype, uint64_t inner, uint64_t outer, uint64_t batch,
                   uint64_t outer_stride_bytes, uint64_t batch_stride_bytes, uint32_t box_inner, uint32_t box_outer);
int* gemm_status_word_device();
int gemm_sm_count();
// 2-CTA (cta_group::2) variant; returns cudaErrorNotSupported when it does not apply
int gemm_launch_2cta(const b200_gemm_desc_t* g, void* d, const void* a, const void* b, cudaStream_t stream,
                     const GemmPlan& plan, const AgParams* ag = nullptr, const RsParams* rs = nullptr);
GemmPlan gemm_plan(const b200_gemm_desc_t* g);
// sums the fp32 partial products of a split-K run and applies bias / activation / accumulate / output cast
int gemm_splitk_reduce(const b200_gemm_desc_t* g, void* d, const float* ws, int splits, cudaStream_t stream);

}  // namespace b200k
