// Caching device allocator for the blackwell backend.
//
// One DeviceAllocator per GPU.  Requests are rounded to 512 B, served from a
// small pool (requests <= 1 MiB, carved out of 2 MiB segments) or a large pool
// (20 MiB segments for requests < 10 MiB, else rounded to 2 MiB), best-fit per
// stream, with split/merge, cross-stream reuse gated by events
// (record_stream), a garbage-collection threshold, a per-process memory
// fraction, private pools that graph capture allocates from, OOM retry after
// releasing cached segments, OOM observers, statistics in torch's key scheme
// and a segment snapshot.  A B200 has 180 GB of HBM3e, so segments above
// 1 GiB are never split further unless max_split_size asks for it and the
// large-segment granularity can be raised (`large_segment_mb`).
//
// The raw memory source is a small table of function pointers so the same
// cache logic runs over cudaMalloc ("native"), cudaMallocManaged ("unified",
// the managed-memory backend), cudaMallocAsync ("cudaMallocAsync"), a user
// plug-in, or plain host malloc ("host": used by the CPU-only unit tests, where
// events complete immediately).
//
// Parity: reference torch_musa/csrc/core/MUSACachingAllocator.h:179-271 and
// MUSACachingAllocator.cpp:45-57,774-1106,1207-1319,1773-1836,2231-2473,
// MUSAAllocatorConfig.cpp:223-296, MUSAUnifiedAllocator.cpp:8-30.
#pragma once

#include "core/Device.h"
#include "core/Stream.h"

#include <c10/core/Allocator.h>

#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>

namespace b200 {
namespace alloc {

using MempoolId = std::pair<uint64_t, uint64_t>;

// Virtual-memory operations behind expandable segments: address space is
// reserved once per (pool, stream) and physical chunks are mapped into it as the
// pool grows, so one segment grows in place instead of the cache collecting
// differently sized cudaMalloc segments that fragment.  The CUDA table uses the
// driver's cuMem* calls; the host table uses mmap/mprotect so the block logic
// is exercised by the CPU tests.
struct VmmOps {
  size_t (*granularity)(int device);
  int (*reserve)(void** va, size_t n, int device);
  int (*release)(void* va, size_t n, int device);
  // Creates `n` bytes of physical memory on `device`, maps them at `va` read/write and returns a handle.
  int (*map)(void* va, size_t n, int device, uint64_t* handle);
  int (*unmap)(void* va, size_t n, int device, uint64_t handle);
  // POSIX file descriptor that another process can import (storage sharing); -1 table entries mean unsupported.
  int (*export_fd)(uint64_t handle, int* fd);
  int (*import_fd)(int fd, void* va, size_t n, int device, uint64_t* handle);
};

struct RawBackend {
  const char* name;
  // All functions are called with `device` current.
  int (*raw_alloc)(void** p, size_t n, int device, cudaStream_t stream);
  int (*raw_free)(void* p, size_t n, int device, cudaStream_t stream);
  int (*mem_info)(int device, size_t* free_b, size_t* total_b);
  // Event hooks; null table entries mean "events complete immediately".
  bool device_events;
  // Null when the memory source cannot grow a segment in place.
  const VmmOps* vmm = nullptr;
};

B200_EXPORT const RawBackend* native_backend();
B200_EXPORT const RawBackend* unified_backend();
B200_EXPORT const RawBackend* async_backend();
B200_EXPORT const RawBackend* host_backend();

struct Config {
  size_t max_split_size = SIZE_MAX;          // bytes; blocks larger than this are not split
  double gc_threshold = 0.0;                 // fraction of the allowed memory that triggers cache GC
  size_t roundup_power2_divisions = 0;       // 0 = off
  size_t large_segment_bytes = 20u << 20;    // segment size for mid-sized requests
  bool expandable_segments = false;          // grow segments in place through the backend's VmmOps
  bool release_lock_on_malloc = false;
  bool pinned_use_host_register = false;
  int pinned_num_register_threads = 1;
  bool pinned_use_background_threads = false;
  std::string backend = "native";            // native | unified | cudaMallocAsync | host
  bool cpu_unified = false;                  // "cpu:unified": CPU allocator hands out managed memory
  bool no_caching = false;                   // PYTORCH_NO_BLACKWELL_MEMORY_CACHING
  bool canary = false;                       // debug: guard bytes behind every allocation, verified when it is freed
};

// Parses "key:value,key:value" (the PYTORCH_BLACKWELL_ALLOC_CONF syntax); throws on unknown keys.
B200_EXPORT Config parse_config(const std::string& s, Config base = Config());
B200_EXPORT const Config& config();
B200_EXPORT void set_config_string(const std::string& s);

struct Stat {
  int64_t current = 0, peak = 0, allocated = 0, freed = 0;
  void inc(int64_t n) { current += n; if (current > peak) peak = current; allocated += n; }
  void dec(int64_t n) { current -= n; freed += n; }
  void reset_accumulated() { allocated = 0; freed = 0; }
  void reset_peak() { peak = current; }
};

enum StatType { kAll = 0, kSmall = 1, kLarge = 2, kNumStatTypes = 3 };

struct DeviceStats {
  Stat allocation[kNumStatTypes], segment[kNumStatTypes], active[kNumStatTypes], inactive_split[kNumStatTypes];
  Stat allocated_bytes[kNumStatTypes], reserved_bytes[kNumStatTypes], active_bytes[kNumStatTypes],
      inactive_split_bytes[kNumStatTypes], requested_bytes[kNumStatTypes];
  Stat oversize_allocations, oversize_segments;
  int64_t num_alloc_retries = 0, num_ooms = 0, num_sync_all_streams = 0, num_device_alloc = 0, num_device_free = 0;
  int64_t max_split_size = 0;
};

struct BlockInfo {
  uintptr_t address = 0;
  size_t size = 0, requested = 0;
  bool allocated = false, active = false;
};
struct SegmentInfo {
  int device = 0;
  uintptr_t address = 0;
  size_t total_size = 0, allocated_size = 0, active_size = 0, requested_size = 0;
  cudaStream_t stream = nullptr;
  bool is_large = false, is_expandable = false;
  uint64_t pool_id_first = 0, pool_id_second = 0;
  std::vector<BlockInfo> blocks;
};

// Block layout of one private pool at a point in time.  Restoring it frees what
// was allocated since and re-creates the blocks that were live then at the
// same addresses (graph trees replay an earlier graph's outputs this way).
struct PoolCheckpoint {
  int device = 0;
  MempoolId pool{0, 0};
  std::vector<SegmentInfo> segments;
};
struct RestoreResult {
  std::vector<void*> freed;      // live before the restore, not live in the checkpoint
  std::vector<void*> allocated;  // live in the checkpoint (whether or not they were live before)
};

struct TraceEntry {
  enum Action { ALLOC, FREE_REQUESTED, FREE_COMPLETED, SEGMENT_ALLOC, SEGMENT_FREE, OOM, SNAPSHOT } action;
  int device;
  uintptr_t addr;
  size_t size;
  cudaStream_t stream;
  uint64_t time_ns;
  std::string stack;  // symbolised caller frames (record_history(..., stacks=true))
};

using OomObserver = std::function<void(int device, size_t requested, size_t total, size_t free_b)>;

class DeviceAllocatorImpl;

// The allocator facade.  One process-wide instance per backend kind.
class B200_EXPORT CachingAllocator final : public c10::Allocator {
 public:
  explicit CachingAllocator(const RawBackend* backend, int num_devices = -1);
  ~CachingAllocator() override;

  // c10::Allocator
  c10::DataPtr allocate(size_t n) override;
  c10::DeleterFnPtr raw_deleter() const override;
  void copy_data(void* dst, const void* src, size_t n) const override;

  void init(int num_devices);
  bool initialized() const { return !devs_.empty(); }
  const RawBackend* backend() const { return backend_; }

  void* raw_alloc(size_t n, int device, cudaStream_t stream);
  void raw_delete(void* p);
  // Marks the block owning `p` as used on `stream`; its reuse waits for that stream.
  void record_stream(const c10::DataPtr& p, int device, cudaStream_t stream);
  void record_stream_ptr(void* p, int device, cudaStream_t stream);
  void empty_cache(int device = -1, MempoolId pool = {0, 0});
  void set_memory_fraction(double f, int device);
  double get_memory_fraction(int device);
  DeviceStats stats(int device);
  void reset_accumulated_stats(int device);
  void reset_peak_stats(int device);
  std::vector<SegmentInfo> snapshot(int device = -1, MempoolId pool = {0, 0});
  void* base_allocation(void* p, size_t* size);
  void mem_info(int device, size_t* free_b, size_t* total_b);
  // Whether `p` lies inside a live block of this allocator (any device).
  bool owns(const void* p, int* device = nullptr);

  // Private pools (graph capture): route allocations whose stream passes `filter` to `pool`.
  void begin_allocate_to_pool(int device, MempoolId pool, std::function<bool(cudaStream_t)> filter);
  void end_allocate_to_pool(int device, MempoolId pool);
  void release_pool(int device, MempoolId pool);
  void create_or_incref_pool(int device, MempoolId pool);
  int pool_use_count(int device, MempoolId pool);

  // Private-pool checkpointing (reference MUSACachingAllocator.cpp:1207-1319 keeps the same pair).
  PoolCheckpoint checkpoint_pool(int device, MempoolId pool);
  RestoreResult restore_pool(int device, const PoolCheckpoint& state);
  // Swaps the deleter of a DataPtr that a restore freed for a no-op, or back for one it re-created.
  static c10::DeleterFnPtr noop_deleter();
  // DataPtr for a pointer that restore_pool() reported as allocated.
  c10::DataPtr adopt(void* p, int device);

  // Expandable segments: file descriptors of the physical chunks behind the allocation holding `p`
  // plus its offset in the first chunk, for another process to map (storage sharing without cudaIpc).
  struct ShareInfo { std::vector<int> fds; size_t chunk_bytes = 0, offset = 0, size = 0; };
  bool share_expandable(void* p, ShareInfo* out);
  // The receiving side: maps imported chunks into fresh address space; `unmap_imported` undoes it.
  void* map_imported(const std::vector<int>& fds, size_t chunk_bytes, int device, std::vector<uint64_t>* handles);
  void unmap_imported(void* va, size_t chunk_bytes, int device, const std::vector<uint64_t>& handles);
  // Re-grants read/write on `device`'s mapped chunks to the GPUs that now have peer access to it.
  void refresh_peer_access(int device);

  // Number of allocations whose guard bytes were found overwritten (option `canary:True`), and the last report.
  int64_t canary_violations() const;
  std::string last_canary_report() const;

  void attach_oom_observer(OomObserver o);
  void record_history(bool enabled, size_t max_entries, bool stacks = false);
  std::vector<TraceEntry> trace(int device);
  static MempoolId new_pool_id(bool user_created);

 private:
  const RawBackend* backend_;
  std::vector<std::unique_ptr<DeviceAllocatorImpl>> devs_;
  friend class DeviceAllocatorImpl;
};

// The allocator currently installed for PrivateUse1 (chosen by the `backend:` option).
B200_EXPORT CachingAllocator* get();
// Installs a pluggable allocator (user malloc/free) in place of the caching one. Only before first use.
B200_EXPORT void install_pluggable(int (*malloc_fn)(void**, size_t, int, cudaStream_t),
                                  int (*free_fn)(void*, size_t, int, cudaStream_t));
B200_EXPORT std::string backend_name();

}  // namespace alloc
}  // namespace b200
