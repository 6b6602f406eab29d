// bf16/fp16 GEMM on paired SMs: tcgen05.mma.cta_group::2.
//
//   D[M,N] (+)= alpha * A[M,K] * B[N,K]^T (+ bias) (act)
//
// A cluster of two CTAs (one per SM of a pair) owns a 256 x BN output tile (BN = 256 in every shipped
// instantiation; the kernel is written for any BN that is a multiple of 128).
// Each CTA stages its own 128 rows of A and its own BN/2 rows of B in 128B-swizzled shared
// memory; one elected thread of the leader CTA issues M256 x BN x K16 instructions that read
// both CTAs' shared memory and write 128 accumulator lanes x BN columns into each CTA's TMEM.
// Against the single-CTA kernel this halves the B traffic per SM (64 instead of 96 bytes of
// operand per tensor-core clock).
//
// Roles per CTA (six warps): warp 0 TMA producer (its loads signal the leader's "full"
// barrier; no cluster multicast is used on any load), warp 1 TMEM allocation and -- in the
// leader only -- MMA issue, warps 2-5 epilogue for the CTA's own 128 rows.  Ring slots and
// accumulators are released to both CTAs with one multicast tcgen05.commit; the epilogues of
// both CTAs hand an accumulator back by arriving on the leader's barrier.
// Tiles are handed out either statically (cluster i takes tiles i, i+74, ...) or by cluster launch control:
// the grid asks for one cluster per tile and a scheduler warp of each running cluster cancels clusters that
// have not started and takes their tiles, so SMs that are busy with another kernel simply get no tiles.
// Every wait is bounded; the CTAs of a pair leave together through a cluster barrier so no
// signal can target the shared memory of a CTA that is gone.
//
// Parity: the reference sends mm/addmm/bmm to a closed vendor library
// (reference torch_musa/csrc/aten/ops/Matmul.cpp:293-335,373-380).
#include "gemm_common.cuh"
#include "comm_common.cuh"

#include <algorithm>
#include <atomic>
#include <cstdlib>

namespace b200k {
namespace {
using namespace gemmdev;

constexpr int BM2 = 256;      // rows per cluster tile
constexpr int BMH = 128;      // rows per CTA
constexpr int BK = 64;
constexpr int kThreads = 224;  // TMA, MMA, 4 epilogue warps, tile scheduler
constexpr uint32_t kTmemCols = 512;

template <int BN>
struct Cfg {
  static constexpr int kBHalf = BN / 2;                   // B rows staged by each CTA
  static constexpr int kATile = BMH * BK * 2;             // 16 KB
  static constexpr int kBTile = kBHalf * BK * 2;          // 16 KB / 8 KB
  static constexpr int kStage = kATile + kBTile;
  static constexpr int kStages = BN == 256 ? 6 : 8;       // 192 KB of ring either way
  static constexpr int kAcc = (int)kTmemCols / BN;        // 2 / 4 accumulators
  static constexpr int kSmem = kStages * kStage + 1024 /*alignment slack*/ + 512 /*barriers*/;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_u32(uint32_t cta_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(cta_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// barrier given as a shared::cluster address (possibly in the peer CTA)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
// Tile load into this CTA's shared memory; completion bytes are credited to a barrier that may live in
// the peer CTA (the pair's leader).
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// One arrival on the barrier at this shared-memory offset in every CTA of the mask, once all MMAs issued so
// far by this thread have completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t cta_mask) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(cta_mask)
      : "memory");
}

// ---- cluster launch control: a running cluster asks the hardware for the coordinates of a cluster of this
// grid that has not started yet and takes over its tile; the answer (16 bytes) is delivered to the same
// shared-memory offset in both CTAs and credited to the mbarrier at the same offset in both.
__device__ __forceinline__ void clc_try_cancel(void* response, uint64_t* bar) {
  asm volatile(
      "clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes.multicast::cluster::all.b128 [%0], [%1];"
      ::"r"(smem_u32(response)), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void clc_decode(const void* response, uint32_t& first_ctaid_x, uint32_t& valid) {
  uint32_t x = 0, y = 0, z = 0, v = 0;
  asm volatile(
      "{\n\t.reg .pred p1;\n\t.reg .b128 r;\n\t"
      "ld.shared.b128 r, [%4];\n\t"
      "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 p1, r;\n\t"
      "selp.u32 %3, 1, 0, p1;\n\t"
      "@p1 clusterlaunchcontrol.query_cancel.get_first_ctaid.v4.b32.b128 {%0, %1, %2, _}, r;\n\t}"
      : "+r"(x), "+r"(y), "+r"(z), "+r"(v)
      : "r"(smem_u32(response))
      : "memory");
  // the next answer is written through the async proxy: order this generic-proxy read before it
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  first_ctaid_x = x;
  valid = v;
}
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar_cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.release.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(bar_cluster_addr),
               "r"(bytes)
               : "memory");
}

constexpr int kClcStages = 3;
constexpr int kClcConsumers = 12;  // leader: TMA, MMA, 4 epilogue warps, scheduler; peer: TMA, 4 epilogue warps

// Per-role cursor over the ring of scheduler answers.
struct TileCursor {
  uint64_t* full;        // this CTA's "answer arrived" barriers
  const uint4* resp;     // this CTA's copy of the answers
  uint32_t empty0;       // shared::cluster address of the leader's "answer consumed" barriers
  int stage;
  uint32_t phase;
};

// Next tile of this cluster.  Static schedule: stride by the number of pairs.  Dynamic schedule: consume one
// scheduler answer.  Returns false when there is no further tile or a bounded wait expired.
__device__ __forceinline__ bool next_tile(TileCursor& c, int dynamic, int& tile, int stride, int total,
                                          volatile int* abort_flag) {
  if (!dynamic) {
    tile += stride;
    return tile < total;
  }
  if (!mbar_wait(&c.full[c.stage], c.phase, abort_flag)) return false;
  uint32_t x, valid;
  clc_decode(&c.resp[c.stage], x, valid);
  mbar_arrive_cluster(c.empty0 + (uint32_t)c.stage * 8u);
  if (++c.stage == kClcStages) { c.stage = 0; c.phase ^= 1; }
  tile = (int)(x >> 1);
  return valid != 0 && tile < total;
}

// ---- all-gather copier: one thread per CTA streams 32 KB chunks peer HBM -> shared memory -> local HBM with
// bulk copies (no multicast), five loads in flight, and publishes a panel flag when a 256-row panel is complete.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void bulk_store_1d(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(gdst), "r"(smem_u32(smem_src)),
               "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// spins until (int)(*p - want) >= 0; false when the wait limit expired or another thread of the CTA gave up
template <bool SYS>
__device__ __forceinline__ bool wait_word(const uint32_t* p, uint32_t want, volatile int* abort_flag,
                                          long long limit = c_wait_cycles) {
  const long long t0 = clock64();
  uint32_t spins = 0;
  while ((int32_t)((SYS ? ld_acquire_sys_u32(p) : ld_acquire_gpu_u32(p)) - want) < 0) {
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > limit) { *abort_flag = 1; return false; }
    }
  }
  return true;
}

constexpr int kAgRing = 6;            // 32 KB slots in the operand ring's shared memory
constexpr uint32_t kAgChunk = 32768;

__device__ void ag_copier(const AgParams& ag, uint8_t* ring, uint64_t* bars, volatile int* abort_flag) {
  const int cc = blockIdx.x, n_cc = 2 * ag.copier_pairs;
  const int W = ag.world, r = ag.rank;
  // 1. tell every peer that my shard is complete (my earlier kernels have finished) and wait for theirs
  __threadfence_system();
  for (int peer = 0; peer < W; ++peer)
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ag.sig[peer] + cc * 16 + r), "r"(ag.epoch) : "memory");
  bool ok = true;
  for (int peer = 0; peer < W && ok; ++peer) ok = wait_word<true>(ag.sig[r] + cc * 16 + peer, ag.epoch, abort_flag, ag.wait_cycles);
  // 2. my panels, own shard first (the GEMM clusters consume panels in the same rotated order)
  const int n_panels = ag.panels_per_shard * W;
  const int chunks_per_panel = (int)(ag.panel_bytes / kAgChunk);
  const int my_panels = ok ? (n_panels - cc + n_cc - 1) / n_cc : 0;
  const long long total = (long long)my_panels * chunks_per_panel;
  auto chunk_addr = [&](long long g, const char*& src, char*& dst, int& panel, bool& last) {
    const int q = cc + (int)(g / chunks_per_panel) * n_cc;
    const int i = (int)(g % chunks_per_panel);
    panel = (q + r * ag.panels_per_shard) % n_panels;
    const int owner = panel / ag.panels_per_shard;
    src = static_cast<const char*>(ag.src[owner]) + (long long)(panel - owner * ag.panels_per_shard) * ag.panel_bytes +
          (long long)i * kAgChunk;
    dst = static_cast<char*>(ag.dst) + (long long)panel * ag.panel_bytes + (long long)i * kAgChunk;
    last = i == chunks_per_panel - 1;
  };
  auto issue_load = [&](long long g) {
    const char* src; char* dst; int panel; bool last;
    chunk_addr(g, src, dst, panel, last);
    const int s = (int)(g % kAgRing);
    mbar_expect_tx(&bars[s], kAgChunk);
    bulk_load_1d(ring + (size_t)s * kAgChunk, src, kAgChunk, &bars[s]);
  };
  long long issued = 0;
  for (; issued < total && issued < kAgRing - 1; ++issued) issue_load(issued);
  for (long long g = 0; g < total && ok; ++g) {
    const int s = (int)(g % kAgRing);
    if (!mbar_wait(&bars[s], (uint32_t)((g / kAgRing) & 1), abort_flag)) { ok = false; break; }
    const char* src; char* dst; int panel; bool last;
    chunk_addr(g, src, dst, panel, last);
    bulk_store_1d(dst, ring + (size_t)s * kAgChunk, kAgChunk);
    if (issued < total) {
      // the slot of chunk g-1 is reused now: its store must have finished reading shared memory
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      issue_load(issued++);
    }
    if (last) {
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // the panel's bytes are in local memory
      asm volatile("fence.proxy.async;" ::: "memory");
      __threadfence();
      asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(ag.flags + panel), "r"(ag.epoch) : "memory");
    }
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  // 3. nobody's shard may be overwritten before every peer has finished pulling from it
  for (int peer = 0; peer < W; ++peer)
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(ag.sig[peer] + cc * 16 + r), "r"(ag.epoch + 1) : "memory");
  for (int peer = 0; peer < W && ok; ++peer) ok = wait_word<true>(ag.sig[r] + cc * 16 + peer, ag.epoch + 1, abort_flag, ag.wait_cycles);
}

// ---- reduce-scatter reducer: all threads of the CTA.  Work items are 8 KB chunks of this rank's own panels;
// per item one thread pulls the chunk from every source rank's partial buffer into shared memory with bulk
// copies (two stages), then all threads add the `world` copies in fp32 and store bf16/fp16 output.
constexpr uint32_t kRsChunk = 8192;

template <typename OutT>
__device__ void rs_reducer(const RsParams& rs, int tiles_n, uint8_t* stage_mem, uint64_t* bars, volatile int* abort_flag) {
  const int cc = blockIdx.x, n_cc = 2 * rs.reducer_pairs;
  const int W = rs.world, r = rs.rank;
  const int chunks_per_panel = (int)(rs.panel_bytes / kRsChunk);
  const long long n_items = (long long)rs.panels_per_shard * chunks_per_panel;
  const uint32_t stage_bytes = (uint32_t)W * kRsChunk;
  int waited_panel = -1;
  auto wait_panel = [&](int p) {
    // every tile of panel p from every source rank has been written (flags live in MY arena)
    const uint32_t* base = rs.flag[r];
    const int per_src = rs.panels_per_shard * tiles_n * 2;
    for (int i = threadIdx.x; i < W * tiles_n * 2; i += blockDim.x) {
      const int src = i / (tiles_n * 2), j = i - src * (tiles_n * 2);
      wait_word<true>(base + src * per_src + p * tiles_n * 2 + j, rs.epoch, abort_flag, rs.wait_cycles);
    }
    __syncthreads();
  };
  auto issue = [&](long long item, int st) {
    const int p = (int)(item / chunks_per_panel), c = (int)(item % chunks_per_panel);
    const long long off = ((long long)(r * rs.panels_per_shard + p)) * rs.panel_bytes + (long long)c * kRsChunk;
    asm volatile("fence.proxy.async;" ::: "memory");   // flag acquires (generic proxy) before the bulk reads
    mbar_expect_tx(&bars[st], stage_bytes);
    for (int s = 0; s < W; ++s) {
      const int src = (r + s) % W;
      bulk_load_1d(stage_mem + (size_t)st * stage_bytes + (size_t)s * kRsChunk, static_cast<const char*>(rs.src[src]) + off,
                   kRsChunk, &bars[st]);
    }
  };
  // item sequence of this CTA: cc, cc + n_cc, ...; the k-th item uses stage k % NS with parity (k / NS) & 1 and is
  // requested NS - 1 items ahead, so NS - 1 stages of peer reads are in flight while one stage is being summed
  // up to 12 stages: bars[0..11] are the ring's "full" and "empty" barriers, adjacent in shared memory and all
  // initialised with one expected arrival; a reducer CTA uses them for nothing else
  const int NS = max(2, min(12, (int)(196608u / stage_bytes)));
  const long long my_items = cc < n_items ? (n_items - cc + n_cc - 1) / n_cc : 0;
  auto request = [&](long long k) {       // all threads: wait for the item's panel, then one thread issues the loads
    const long long item = cc + k * n_cc;
    const int pn = (int)(item / chunks_per_panel);
    if (pn != waited_panel) { wait_panel(pn); waited_panel = pn; }
    if (threadIdx.x == 0 && !*abort_flag) issue(item, (int)(k % NS));
  };
  long long requested = 0;
  for (; requested < my_items && requested < NS - 1; ++requested) request(requested);
  for (long long k = 0; k < my_items; ++k) {
    if (*abort_flag) break;
    const int st = (int)(k % NS);
    // stage (k + NS - 1) % NS held item k - 1, which every thread finished reading before the barrier below
    if (requested < my_items) request(requested++);
    if (!mbar_wait(&bars[st], (uint32_t)((k / NS) & 1), abort_flag)) break;
    const long long item = cc + k * n_cc;
    const int p = (int)(item / chunks_per_panel), c = (int)(item % chunks_per_panel);
    OutT* out = reinterpret_cast<OutT*>(static_cast<char*>(rs.out) + (long long)p * rs.panel_bytes + (long long)c * kRsChunk);
    const uint8_t* sm = stage_mem + (size_t)st * stage_bytes;
    for (int v = threadIdx.x; v < (int)(kRsChunk / 16); v += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = 0.f;
      for (int s = 0; s < W; ++s) {
        const Vec16<OutT> x = *reinterpret_cast<const Vec16<OutT>*>(sm + (size_t)s * kRsChunk + (size_t)v * 16);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += ToF<OutT>::to(x.v[e]);
      }
      Vec16<OutT> o;
#pragma unroll
      for (int e = 0; e < 8; ++e) o.v[e] = ToF<OutT>::from(acc[e]);
      st16(out + (size_t)v * 8, o);
    }
    __syncthreads();   // the stage may be refilled
  }
  __syncthreads();
  // peers may overwrite their partial buffers only after everybody has finished pulling
  if (threadIdx.x == 0) {
    __threadfence_system();
    for (int peer = 0; peer < W; ++peer)
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(rs.sig[peer] + cc * 16 + r), "r"(rs.epoch + 1) : "memory");
    bool ok = !*abort_flag;
    for (int peer = 0; peer < W && ok; ++peer) ok = wait_word<true>(rs.sig[r] + cc * 16 + peer, rs.epoch + 1, abort_flag, rs.wait_cycles);
  }
  __syncthreads();
}

template <typename OutT, bool A_KMAJOR, bool B_KMAJOR, int BN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 OutT* __restrict__ d, const Params p, const int dynamic, const AgParams ag, const RsParams rs) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  // Both CTAs of the pair must use identical shared-memory offsets: the dynamic segment starts at the same
  // offset in every CTA of a launch, so the same round-up yields the same layout.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* smem_a = smem;
  uint8_t* smem_b = smem + C::kStages * C::kATile;
  uint8_t* ctrl = smem + C::kStages * C::kStage;
  uint4* clc_resp = reinterpret_cast<uint4*>(ctrl);                        // [kClcStages] 16-byte answers
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctrl + 16 * kClcStages);
  uint64_t* full_bar = bars;                          // [kStages]  used in the leader
  uint64_t* empty_bar = bars + C::kStages;            // [kStages]  one per CTA
  uint64_t* tfull_bar = bars + 2 * C::kStages;        // [kAcc]     one per CTA
  uint64_t* tempty_bar = tfull_bar + C::kAcc;         // [kAcc]     used in the leader
  uint64_t* clc_full = tempty_bar + C::kAcc;          // [kClcStages] one per CTA
  uint64_t* clc_empty = clc_full + kClcStages;        // [kClcStages] used in the leader
  uint64_t* throttle_bar = clc_empty + kClcStages;    // leader: the producer started another tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(throttle_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  // clusters [0, n_copiers) do not multiply: they assemble the A operand (all-gather) or reduce the partial
  // products (reduce-scatter)
  const int n_copiers = ag.enabled ? ag.copier_pairs : (rs.enabled ? rs.reducer_pairs : 0);
  const bool copier = (int)(blockIdx.x >> 1) < n_copiers;
  const int n_pairs = (int)(gridDim.x >> 1) - n_copiers;
  const int k_blocks = (p.k + BK - 1) / BK;
  const int tiles_per_batch = p.tiles_m * p.tiles_n;
  const int tiles_all_batches = tiles_per_batch * p.batch;
  const int total_tiles = tiles_all_batches * p.splits;
  // a copier cluster multiplies nothing: giving it a first tile beyond the end idles all of its GEMM roles
  const int pair = copier ? total_tiles : (int)(blockIdx.x >> 1) - n_copiers;
  // with gathered A the m-tiles are visited own shard first, in the order the copiers deliver the panels
  // reduce-scatter: the other ranks' panels first (the next rank's first), the own panels last
  const int m_rot = ag.enabled ? ag.rank * ag.panels_per_shard
                               : (rs.enabled ? ((rs.rank + 1) % rs.world) * rs.panels_per_shard : 0);

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full_bar[s], 1);   // the leader's expect_tx arrival; bytes come from both CTAs
      mbar_init(&empty_bar[s], 1);  // one multicast commit
    }
    for (int s = 0; s < C::kAcc; ++s) {
      mbar_init(&tfull_bar[s], 1);
      mbar_init(&tempty_bar[s], 8);  // four epilogue warps in each of the two CTAs
    }
    for (int s = 0; s < kClcStages; ++s) {
      mbar_init(&clc_full[s], 1);
      mbar_init(&clc_empty[s], kClcConsumers);
    }
    mbar_init(throttle_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // peer barriers initialised and peer TMEM allocated before anything is signalled
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  TileCursor cur;
  cur.full = clc_full;
  cur.resp = clc_resp;
  cur.empty0 = mapa_u32(smem_u32(&clc_empty[0]), 0);
  cur.stage = 0;
  cur.phase = 0;

  if (copier && rs.enabled) rs_reducer<OutT>(rs, p.tiles_n, smem_a, full_bar, abort_flag);   // whole CTA

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (copier) {
      if (lane == 0 && ag.enabled) ag_copier(ag, smem_a, full_bar, abort_flag);
    } else if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const uint32_t full0 = mapa_u32(smem_u32(&full_bar[0]), 0);  // the leader's ring of "full" barriers
      int tile = pair;
      bool more = tile < total_tiles;
      while (more && ok) {
        if (dynamic && leader) mbar_arrive(throttle_bar);  // lets the scheduler ask for the tile after this one
        const int split = tile / tiles_all_batches;
        const int tb = tile - split * tiles_all_batches;
        const int b = tb / tiles_per_batch;
        const int r = tb - b * tiles_per_batch;
        const int kb0 = split * p.kb_per_split;
        const int kb1 = min(k_blocks, kb0 + p.kb_per_split);
        int mt_raw, nt;
        decode_tile(r, p.tiles_m, p.tiles_n, p.group_m, mt_raw, nt);
        const int mt = (mt_raw + m_rot) % p.tiles_m;
        const int m0 = mt * BM2 + (int)rank * BMH;
        const int n0 = nt * BN + (int)rank * C::kBHalf;
        if (ag.enabled) {
          // the 256-row panel of this tile must have been assembled by a copier CTA of this launch
          if (!wait_word<false>(ag.flags + mt, ag.epoch, abort_flag, ag.wait_cycles)) { ok = false; break; }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag)) { ok = false; break; }
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * C::kStage);
          const uint32_t fb = full0 + (uint32_t)stage * 8u;
          uint8_t* sa = smem_a + stage * C::kATile;
          uint8_t* sb = smem_b + stage * C::kBTile;
          const int k0 = kb * BK;
          if constexpr (A_KMAJOR) {
            tma_load_3d_pair(sa, &tmap_a, fb, k0, m0, b);
          } else {
            tma_load_3d_pair(sa, &tmap_a, fb, m0, k0, b);
            tma_load_3d_pair(sa + 8192, &tmap_a, fb, m0 + 64, k0, b);
          }
          if constexpr (B_KMAJOR) {
            tma_load_3d_pair(sb, &tmap_b, fb, k0, n0, b);
          } else {
#pragma unroll
            for (int q = 0; q < C::kBHalf / 64; ++q) tma_load_3d_pair(sb + q * 8192, &tmap_b, fb, n0 + q * 64, k0, b);
          }
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        more = next_tile(cur, dynamic, tile, n_pairs, total_tiles, abort_flag);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      int tile = pair;
      bool more = tile < total_tiles;
      while (more && ok) {
        const int kb0 = (tile / tiles_all_batches) * p.kb_per_split;
        const int kb1 = min(k_blocks, kb0 + p.kb_per_split);
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem_a + stage * C::kATile);
          const uint32_t sb = smem_u32(smem_b + stage * C::kBTile);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk) {
            const uint64_t adesc = A_KMAJOR ? make_desc(sa + kk * 32, 16, 1024) : make_desc(sa + kk * 2048, 8192, 1024);
            const uint64_t bdesc = B_KMAJOR ? make_desc(sb + kk * 32, 16, 1024) : make_desc(sb + kk * 2048, 8192, 1024);
            umma_f16_pair(tmem_d, adesc, bdesc, p.idesc, (kb > kb0 || kk != 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[stage], 3);  // frees this slot in both CTAs
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(&tfull_bar[acc], 3);  // accumulator complete in both CTAs
        if (++acc == C::kAcc) { acc = 0; acc_phase ^= 1; }
        more = next_tile(cur, dynamic, tile, n_pairs, total_tiles, abort_flag);
      }
    }
    __syncwarp();
  } else if (warp == 6) {
    // ------------------------------------------------------------ tile scheduler (leader CTA, dynamic schedule)
    if (dynamic && leader && lane == 0 && pair < total_tiles) {
      const uint32_t peer_full0 = mapa_u32(smem_u32(&clc_full[0]), 1);
      uint32_t tphase = 0;
      bool valid = true;
      // One query in flight at a time: a query may only follow an answer that named a tile.
      while (valid) {
        if (!mbar_wait(throttle_bar, tphase, abort_flag)) break;  // the producer has started the current tile
        tphase ^= 1;
        if (!mbar_wait(&clc_empty[cur.stage], cur.phase ^ 1, abort_flag)) break;  // every role has read the old answer
        mbar_expect_tx(&clc_full[cur.stage], 16);
        mbar_expect_tx_cluster(peer_full0 + (uint32_t)cur.stage * 8u, 16);
        clc_try_cancel(&clc_resp[cur.stage], &clc_full[cur.stage]);
        int unused_tile = 0;
        valid = next_tile(cur, 1, unused_tile, 0, total_tiles, abort_flag);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const uint32_t tempty0 = mapa_u32(smem_u32(&tempty_bar[0]), 0);
    const bool vec_ok = (p.ldd % (16 / (int)sizeof(OutT)) == 0) && ((reinterpret_cast<uintptr_t>(d) & 15) == 0) &&
                        (p.stride_d % (16 / (int)sizeof(OutT)) == 0);
    int tile = pair;
    bool more = tile < total_tiles;
    while (more) {
      const int split = tile / tiles_all_batches;
      const int tb = tile - split * tiles_all_batches;
      const int b = tb / tiles_per_batch;
      const int r = tb - b * tiles_per_batch;
      int mt_raw, nt;
      decode_tile(r, p.tiles_m, p.tiles_n, p.group_m, mt_raw, nt);
      const int mt_e = (mt_raw + m_rot) % p.tiles_m;
      const int m0 = mt_e * BM2 + (int)rank * BMH;
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
      if (rs.enabled) {
        // this CTA's half of the tile is in the partial buffer: tell the owner of the row panel
        __threadfence_system();
        asm volatile("bar.sync 1, 128;" ::: "memory");   // the four epilogue warps
        if (warp == 2 && lane == 0) {
          const int owner = mt_e / rs.panels_per_shard, pin = mt_e - owner * rs.panels_per_shard;
          uint32_t* f = rs.flag[owner] + (((size_t)rs.rank * rs.panels_per_shard + pin) * p.tiles_n + nt) * 2 + rank;
          asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(rs.epoch) : "memory");
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty0 + (uint32_t)acc * 8u);  // hand the accumulator back to the leader
      if (++acc == C::kAcc) { acc = 0; acc_phase ^= 1; }
      // lane 0 reads the scheduler's answer for the whole warp
      int next = tile;
      int go = 0;
      if (lane == 0) go = next_tile(cur, dynamic, next, n_pairs, total_tiles, abort_flag) ? 1 : 0;
      tile = __shfl_sync(0xffffffffu, next, 0);
      more = __shfl_sync(0xffffffffu, go, 0) != 0;
    }
  }

  // A CTA that gave up on a wait may still have tile loads in flight towards its shared memory: give them
  // a bounded moment to land before the memory is released.
  if (*abort_flag && threadIdx.x == 0) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // no CTA of the pair leaves while the other may still signal it
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
}

// ------------------------------------------------------------------ host side
template <typename OutT, int BN>
int launch_pair(const b200_gemm_desc_t* g, void* d, const void* a, const void* b, cudaStream_t stream,
                const GemmPlan& plan, const AgParams* agp, const RsParams* rsp) {
  AgParams ag{};
  if (agp) ag = *agp;
  RsParams rs{};
  if (rsp) rs = *rsp;
  const int dynamic = (ag.enabled || rs.enabled) ? 0 : plan.dynamic;   // helper and GEMM clusters must all be resident
  using C = Cfg<BN>;
  CUtensorMap ma, mb;
  const uint64_t esz = 2;
  const uint64_t batch = (uint64_t)std::max(g->batch, 1);
  bool ok;
  if (g->a_kmajor)
    ok = gemm_make_map(&ma, a, g->in_dtype, (uint64_t)g->k, (uint64_t)g->m, batch, (uint64_t)g->lda * esz,
                       (uint64_t)g->stride_a * esz, BK, BMH);
  else
    ok = gemm_make_map(&ma, a, g->in_dtype, (uint64_t)g->m, (uint64_t)g->k, batch, (uint64_t)g->lda * esz,
                       (uint64_t)g->stride_a * esz, 64, BK);
  if (!ok) return (int)cudaErrorNotSupported;
  if (g->b_kmajor)
    ok = gemm_make_map(&mb, b, g->in_dtype, (uint64_t)g->k, (uint64_t)g->n, batch, (uint64_t)g->ldb * esz,
                       (uint64_t)g->stride_b * esz, BK, C::kBHalf);
  else
    ok = gemm_make_map(&mb, b, g->in_dtype, (uint64_t)g->n, (uint64_t)g->k, batch, (uint64_t)g->ldb * esz,
                       (uint64_t)g->stride_b * esz, 64, BK);
  if (!ok) return (int)cudaErrorNotSupported;

  Params p;
  p.m = g->m; p.n = g->n; p.k = g->k;
  p.batch = (int)batch;
  p.tiles_m = (g->m + BM2 - 1) / BM2;
  p.tiles_n = (g->n + BN - 1) / BN;
  p.ldd = g->ldd;
  p.stride_d = g->stride_d;
  p.bias = g->bias;
  p.bias_f32 = g->bias_dtype == B200_F32;
  p.act = g->act;
  p.accumulate = g->accumulate;
  p.alpha = g->alpha;
  // instruction descriptor: fp32 accumulate, A/B format, majors, N>>3, M>>4 (M counts both CTAs)
  const uint32_t fmt = g->in_dtype == B200_BF16 ? 1u : 0u;
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((g->a_kmajor ? 0u : 1u) << 15) | ((g->b_kmajor ? 0u : 1u) << 16) |
            ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM2 >> 4) << 24);
  p.status = gemm_status_word_device();
  p.splits = plan.splits;
  p.kb_per_split = plan.kb_per_split;
  p.split_stride = (int64_t)g->m * g->n;
  p.group_m = gemm_group_m(BM2, g->m, plan.splits > 1 ? plan.kb_per_split * BK : g->k, !g->a_kmajor && !g->b_kmajor);

  const int total = p.tiles_m * p.tiles_n * p.batch * p.splits;
  const int pairs = std::max(1, gemm_sm_count() / 2);
  // static schedule: one resident cluster per SM pair strides over the tiles; dynamic schedule: one cluster
  // per tile is requested and the clusters that run take over the tiles of those that have not started
  int grid = dynamic ? 2 * total : 2 * std::min(total, pairs);
  if (ag.enabled) grid = 2 * (ag.copier_pairs + std::min(total, std::max(1, pairs - ag.copier_pairs)));
  if (rs.enabled) grid = 2 * (rs.reducer_pairs + std::min(total, std::max(1, pairs - rs.reducer_pairs)));

#define GEMM2_GO(AK, BKM)                                                                                        \
  do {                                                                                                           \
    static bool attr_set = false;                                                                                \
    auto kern = gemm_pair_kernel<OutT, AK, BKM, BN>;                                                             \
    if (!attr_set) {                                                                                             \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmem);         \
      if (e != cudaSuccess) return (int)e;                                                                       \
      attr_set = true;                                                                                           \
    }                                                                                                            \
    kern<<<grid, kThreads, C::kSmem, stream>>>(ma, mb, (OutT*)d, p, dynamic, ag, rs);                                            \
  } while (0)

  if (g->a_kmajor && g->b_kmajor) GEMM2_GO(true, true);
  else if (g->a_kmajor && !g->b_kmajor) GEMM2_GO(true, false);
  else if (!g->a_kmajor && g->b_kmajor) GEMM2_GO(false, true);
  else GEMM2_GO(false, false);
#undef GEMM2_GO
  B200K_LAUNCH_RET();
}

// 0 = cost model, 1 = single CTA 128x256, 2 = SM pair 256x256 static schedule, 3 = SM pair 256x256 dynamic schedule
std::atomic<int> g_forced_config{[] {
  const char* e = std::getenv("B200_GEMM_CONFIG");
  return e ? std::atoi(e) : 0;
}()};

// The dynamic (cluster launch control) schedule is what the cost model picks unless B200_GEMM_DYNAMIC=0: with a
// static schedule a CTA that cannot become resident (its SM is held by a communication kernel) keeps its share
// of the tiles waiting, so one busy SM stretches the whole GEMM to the length of the other kernel.
const bool g_dynamic_default = [] {
  const char* e = std::getenv("B200_GEMM_DYNAMIC");
  return !(e && e[0] == '0');
}();

std::atomic<bool> g_splitk{[] {
  const char* e = std::getenv("B200_GEMM_SPLITK");
  return !(e && e[0] == '0');
}()};

inline long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }

}  // namespace

int gemm_forced_config_exchange(int c) { return g_forced_config.exchange(c); }

// Chooses the kernel family and the split-K factor.
// Family: waves x per-wave cost; per wave the pair kernel is ~15% cheaper (measured 1.42-1.54 against 1.22-1.43
// PFLOP/s on 4096-row bf16 problems) because each SM reads half of B.  256x128 pair tiles were measured too and
// rejected: an N=128 instruction is no faster per column than N=256, so they ran at 0.7-0.98 PFLOP/s.
// Split-K: when the output has fewer tiles than half the machine and K is long (weight gradients of
// convolutions and of small linear layers: K = batch x pixels), K is cut so that every SM (pair) gets a slice.
GemmPlan gemm_plan(const b200_gemm_desc_t* g) {
  const int forced = g_forced_config.load(std::memory_order_relaxed);
  const long long batch = std::max(g->batch, 1);
  const int sms = gemm_sm_count();
  const int pairs = std::max(1, sms / 2);
  int choice = forced;
  if (choice == 0) {
    choice = 1;
    if (g->m > 128) {  // with M <= 128 the second CTA of a pair would only multiply padding
      const long long t1 = ceil_div_ll(g->m, 128) * ceil_div_ll(g->n, 256) * batch;
      const long long t2 = ceil_div_ll(g->m, 256) * ceil_div_ll(g->n, 256) * batch;
      const double c1 = (double)ceil_div_ll(t1, sms) * 1.15;
      const double c2 = (double)ceil_div_ll(t2, pairs);
      if (c2 <= c1) choice = g_dynamic_default ? 3 : 2;
    }
  }
  GemmPlan plan;
  plan.pair = choice == 2 || choice == 3;
  plan.dynamic = choice == 3;
  const bool tf32 = g->in_dtype == B200_F32;  // fp32 operands: single-CTA kernel, 32 elements per K block, no split
  if (tf32) plan.pair = plan.dynamic = false;
  const int k_blocks = (g->k + (tf32 ? 32 : BK) - 1) / (tf32 ? 32 : BK);
  plan.splits = 1;
  plan.kb_per_split = k_blocks;
  if (batch == 1 && !tf32 && g_splitk.load(std::memory_order_relaxed)) {
    const long long tiles = ceil_div_ll(g->m, plan.pair ? 256 : 128) * ceil_div_ll(g->n, 256);
    const long long units = plan.pair ? pairs : sms;
    if (tiles * 2 <= units && k_blocks >= 32) {
      long long s = std::min<long long>(units / tiles, k_blocks / 8);
      s = std::min<long long>(s, 256);
      if (s > 1) {
        plan.kb_per_split = (int)ceil_div_ll(k_blocks, s);
        plan.splits = (int)ceil_div_ll(k_blocks, plan.kb_per_split);  // no empty split
      }
    }
  }
  return plan;
}

int gemm_launch_2cta(const b200_gemm_desc_t* g, void* d, const void* a, const void* b, cudaStream_t stream,
                     const GemmPlan& plan, const AgParams* ag, const RsParams* rs) {
  switch (g->out_dtype) {
    case B200_BF16: return launch_pair<__nv_bfloat16, 256>(g, d, a, b, stream, plan, ag, rs);
    case B200_F16: return launch_pair<__half, 256>(g, d, a, b, stream, plan, ag, rs);
    case B200_F32: return launch_pair<float, 256>(g, d, a, b, stream, plan, ag, rs);
    default: return (int)cudaErrorNotSupported;
  }
}

// ------------------------------------------------------------------ split-K reduction
template <typename OutT>
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ ws, OutT* __restrict__ d, int m, int n, int64_t ldd, int splits,
                     const void* __restrict__ bias, int bias_f32, int act, int accumulate) {
  const int64_t total = (int64_t)m * n;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    float v = 0.f;
    for (int s = 0; s < splits; ++s) v += ws[(int64_t)s * total + i];
    const int64_t r = i / n;
    const int c = (int)(i - r * n);
    if (bias) v += bias_f32 ? reinterpret_cast<const float*>(bias)[c] : ToF<OutT>::to(reinterpret_cast<const OutT*>(bias)[c]);
    if (act) v = apply_act(v, act);
    OutT* o = d + r * ldd + c;
    if (accumulate) v += ToF<OutT>::to(*o);
    *o = ToF<OutT>::from(v);
  }
}

int gemm_splitk_reduce(const b200_gemm_desc_t* g, void* d, const float* ws, int splits, cudaStream_t stream) {
  const int64_t total = (int64_t)g->m * g->n;
  const int grid = (int)std::min<int64_t>((total + 255) / 256, (int64_t)gemm_sm_count() * 8);
  const int bias_f32 = g->bias_dtype == B200_F32;
  switch (g->out_dtype) {
    case B200_BF16:
      splitk_reduce_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(ws, (__nv_bfloat16*)d, g->m, g->n, g->ldd, splits,
                                                                    g->bias, bias_f32, g->act, g->accumulate);
      break;
    case B200_F16:
      splitk_reduce_kernel<__half><<<grid, 256, 0, stream>>>(ws, (__half*)d, g->m, g->n, g->ldd, splits, g->bias,
                                                             bias_f32, g->act, g->accumulate);
      break;
    case B200_F32:
      splitk_reduce_kernel<float><<<grid, 256, 0, stream>>>(ws, (float*)d, g->m, g->n, g->ldd, splits, g->bias,
                                                            bias_f32, g->act, g->accumulate);
      break;
    default: return (int)cudaErrorNotSupported;
  }
  B200K_LAUNCH_RET();
}

}  // namespace b200k

// Pins the tile configuration for every later launch of this process (0 returns to the cost model).
extern "C" int b200_gemm_force_config(int config) {
  if (config < 0 || config > 3) return -1;
  return b200k::gemm_forced_config_exchange(config);
}

// The pipeline waits of a launch that also waits for other ranks must not give up before the cross-rank waits do:
// raise this translation unit's limit to the collective limit on the current device (once per change).
static int sync_wait_limit(long long want, cudaStream_t stream) {
  static std::atomic<long long> applied[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
  if (want < b200k::kWaitCycles) want = b200k::kWaitCycles;
  if (applied[dev].load(std::memory_order_relaxed) == want) return 0;
  cudaError_t e = cudaMemcpyToSymbolAsync(b200k::c_wait_cycles, &want, sizeof(want), 0, cudaMemcpyHostToDevice, stream);
  if (e == cudaSuccess) applied[dev].store(want, std::memory_order_relaxed);
  return (int)e;
}

// all-gather -> GEMM in one launch.  D[M, N] = gather_rows(A shards)[M, K] x B[N, K]^T with M = world * shard
// rows; every rank's shard lives at `shard_off` of its arena; a_full [M, K] and flags [M / 256] are local
// (flags persistent, zero-initialised once).  Consumes epochs `epoch` and `epoch + 1` of the arena's pad.
extern "C" int b200_gemm_allgather(const b200_gemm_desc_t* g, const b200_symm_t* s, int64_t shard_off, void* a_full,
                                   uint32_t* flags, uint32_t epoch, int copier_pairs, void* d, const void* b,
                                   cudaStream_t stream) {
  using namespace b200k;
  if (!g->a_kmajor || g->batch > 1 || s->world < 2 || s->world > 16 || g->m % (256 * s->world) != 0 ||
      g->k % 64 != 0 || g->lda != g->k || (shard_off & 15) || copier_pairs < 1 || copier_pairs > 16 ||
      (reinterpret_cast<uintptr_t>(a_full) & 15))
    return (int)cudaErrorNotSupported;
  if (g->in_dtype != B200_BF16 && g->in_dtype != B200_F16) return (int)cudaErrorNotSupported;
  if (copier_pairs * 2 >= gemm_sm_count() / 2) return (int)cudaErrorNotSupported;
  AgParams ag{};
  ag.enabled = 1;
  ag.wait_cycles = commdev::peer_wait_cycles();
  ag.world = s->world;
  ag.rank = s->rank;
  ag.copier_pairs = copier_pairs;
  ag.panels_per_shard = g->m / s->world / 256;
  ag.panel_bytes = (int64_t)256 * g->k * 2;
  for (int r = 0; r < s->world; ++r) {
    ag.src[r] = static_cast<const char*>(s->bufs[r]) + shard_off;
    ag.sig[r] = s->sigs[r];
  }
  ag.dst = a_full;
  ag.flags = flags;
  ag.epoch = epoch;
  if (int e = sync_wait_limit(ag.wait_cycles, stream)) return e;
  GemmPlan plan;
  plan.pair = 1;
  plan.dynamic = 0;
  plan.splits = 1;
  plan.kb_per_split = (g->k + BK - 1) / BK;
  return gemm_launch_2cta(g, d, a_full, b, stream, plan, &ag);
}

// GEMM -> reduce-scatter in one launch.  out[M / world, N] = rows `rank` of sum over ranks of A_r[M, K_r] x B_r[N, K_r]^T.
// The partial product goes to `partial_off` of the arena ([M, N], output dtype), the flag table to `flag_off`
// (world * M/256/world * N/256 * 2 words, zeroed once).  Consumes epochs `epoch` and `epoch + 1`.
extern "C" int b200_gemm_reduce_scatter(const b200_gemm_desc_t* g, const b200_symm_t* s, int64_t partial_off,
                                        int64_t flag_off, uint32_t epoch, int reducer_pairs, void* out, const void* a,
                                        const void* b, cudaStream_t stream) {
  using namespace b200k;
  if (g->batch > 1 || s->world < 2 || s->world > 8 || g->m % (256 * s->world) != 0 || g->n % 256 != 0 ||
      (partial_off & 1023) || (flag_off & 15) || reducer_pairs < 1 || reducer_pairs > 16 || g->ldd != g->n ||
      g->bias || g->act || g->accumulate || (reinterpret_cast<uintptr_t>(out) & 15))
    return (int)cudaErrorNotSupported;
  if ((g->in_dtype != B200_BF16 && g->in_dtype != B200_F16) || g->out_dtype != g->in_dtype) return (int)cudaErrorNotSupported;
  if (reducer_pairs * 2 >= gemm_sm_count() / 2) return (int)cudaErrorNotSupported;
  RsParams rs{};
  rs.enabled = 1;
  rs.wait_cycles = commdev::peer_wait_cycles();
  rs.world = s->world;
  rs.rank = s->rank;
  rs.reducer_pairs = reducer_pairs;
  rs.panels_per_shard = g->m / s->world / 256;
  rs.panel_bytes = (int64_t)256 * g->n * 2;
  for (int r = 0; r < s->world; ++r) {
    rs.src[r] = static_cast<const char*>(s->bufs[r]) + partial_off;
    rs.flag[r] = reinterpret_cast<uint32_t*>(static_cast<char*>(s->bufs[r]) + flag_off);
    rs.sig[r] = s->sigs[r];
  }
  rs.out = out;
  rs.epoch = epoch;
  if (int e = sync_wait_limit(rs.wait_cycles, stream)) return e;
  GemmPlan plan;
  plan.pair = 1;
  plan.dynamic = 0;
  plan.splits = 1;
  plan.kb_per_split = (g->k + BK - 1) / BK;
  void* partial = static_cast<char*>(s->bufs[s->rank]) + partial_off;
  return gemm_launch_2cta(g, partial, a, b, stream, plan, nullptr, &rs);
}
