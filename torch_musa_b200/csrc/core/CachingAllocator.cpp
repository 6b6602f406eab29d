#include "core/CachingAllocator.h"

#include <c10/util/Exception.h>
#include <c10/util/irange.h>

#include <algorithm>
#include <chrono>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <mutex>
#include <set>
#include <sstream>
#include <unordered_map>
#include <unordered_set>

namespace b200 {
namespace alloc {

static size_t g_host_in_use = 0;  // bytes handed out by the "host" test backend

namespace {

constexpr size_t kMinBlock = 512;          // every size is a multiple of this
constexpr size_t kSmallSize = 1u << 20;    // requests up to 1 MiB go to the small pool
constexpr size_t kSmallBuffer = 2u << 20;  // small-pool segments
constexpr size_t kMinLargeAlloc = 10u << 20;
constexpr size_t kRoundLarge = 2u << 20;
constexpr size_t kHugeNoSplit = 1ull << 30;  // remainder of >1 GiB segments stays whole unless asked

uint64_t now_ns() {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(std::chrono::steady_clock::now().time_since_epoch())
      .count();
}

// ---------------------------------------------------------------- backends
int native_alloc(void** p, size_t n, int, cudaStream_t) { return (int)cudaMalloc(p, n); }
int native_free(void* p, size_t, int, cudaStream_t) { return (int)cudaFree(p); }
int cuda_mem_info(int, size_t* f, size_t* t) { return (int)cudaMemGetInfo(f, t); }
int unified_alloc(void** p, size_t n, int device, cudaStream_t) {
  cudaError_t e = cudaMallocManaged(p, n, cudaMemAttachGlobal);
  if (e == cudaSuccess) {
    // Prefer residency on the allocating GPU; the host may still touch the pages.
    cudaMemLocation loc{};
    loc.type = cudaMemLocationTypeDevice;
    loc.id = device;
    (void)loc;
    cudaMemAdvise(*p, n, cudaMemAdviseSetPreferredLocation, device);
    (void)cudaGetLastError();
  }
  return (int)e;
}
int async_alloc(void** p, size_t n, int, cudaStream_t s) { return (int)cudaMallocAsync(p, n, s); }
int async_free(void* p, size_t, int, cudaStream_t s) { return (int)cudaFreeAsync(p, s); }
int host_alloc(void** p, size_t n, int, cudaStream_t) {
  *p = nullptr;
  // An artificial ceiling lets the tests exercise the OOM/retry path without a GPU.
  static const size_t cap = [] {
    const char* e = std::getenv("B200_HOST_BACKEND_CAP_MB");
    return e ? (size_t)std::atoll(e) << 20 : (size_t)1 << 40;
  }();
  if (g_host_in_use + n > cap) return (int)cudaErrorMemoryAllocation;
  if (posix_memalign(p, 512, n) != 0) return (int)cudaErrorMemoryAllocation;
  g_host_in_use += n;
  return 0;
}
int host_free(void* p, size_t n, int, cudaStream_t) {
  g_host_in_use -= n;
  free(p);
  return 0;
}
int host_mem_info(int, size_t* f, size_t* t) {
  *t = (size_t)1 << 34;
  *f = *t > g_host_in_use ? *t - g_host_in_use : 0;
  return 0;
}

const RawBackend kNative{"native", native_alloc, native_free, cuda_mem_info, true};
const RawBackend kUnified{"unified", unified_alloc, native_free, cuda_mem_info, true};
const RawBackend kAsync{"cudaMallocAsync", async_alloc, async_free, cuda_mem_info, true};
const RawBackend kHost{"host", host_alloc, host_free, host_mem_info, false};
RawBackend g_plug{"pluggable", nullptr, nullptr, cuda_mem_info, true};

}  // namespace

const RawBackend* native_backend() { return &kNative; }
const RawBackend* unified_backend() { return &kUnified; }
const RawBackend* async_backend() { return &kAsync; }
const RawBackend* host_backend() { return &kHost; }

// ------------------------------------------------------------------ config
static std::string trim(const std::string& s) {
  size_t a = s.find_first_not_of(" \t\n"), b = s.find_last_not_of(" \t\n");
  return a == std::string::npos ? "" : s.substr(a, b - a + 1);
}
static bool parse_bool(const std::string& k, const std::string& v) {
  if (v == "True" || v == "true" || v == "1") return true;
  if (v == "False" || v == "false" || v == "0") return false;
  TORCH_CHECK(false, "allocator config: expected True/False for ", k, ", got '", v, "'");
}

Config parse_config(const std::string& s, Config c) {
  std::stringstream ss(s);
  std::string item;
  while (std::getline(ss, item, ',')) {
    item = trim(item);
    if (item.empty()) continue;
    auto pos = item.find(':');
    TORCH_CHECK(pos != std::string::npos, "allocator config: expected key:value, got '", item, "'");
    std::string k = trim(item.substr(0, pos)), v = trim(item.substr(pos + 1));
    if (k == "max_split_size_mb") {
      long long mb = std::atoll(v.c_str());
      TORCH_CHECK(mb > 20, "allocator config: max_split_size_mb must be larger than 20");
      c.max_split_size = (size_t)mb << 20;
    } else if (k == "garbage_collection_threshold") {
      double t = std::atof(v.c_str());
      TORCH_CHECK(t > 0.0 && t < 1.0, "allocator config: garbage_collection_threshold must be in (0,1)");
      c.gc_threshold = t;
    } else if (k == "roundup_power2_divisions") {
      long long d = std::atoll(v.c_str());
      TORCH_CHECK(d > 0 && (d & (d - 1)) == 0, "allocator config: roundup_power2_divisions must be a power of two");
      c.roundup_power2_divisions = (size_t)d;
    } else if (k == "large_segment_mb") {
      long long mb = std::atoll(v.c_str());
      TORCH_CHECK(mb >= 20 && mb % 2 == 0, "allocator config: large_segment_mb must be an even number >= 20");
      c.large_segment_bytes = (size_t)mb << 20;
    } else if (k == "backend") {
      TORCH_CHECK(v == "native" || v == "unified" || v == "cudaMallocAsync" || v == "host",
                  "allocator config: unknown backend '", v, "' (native|unified|cudaMallocAsync|host)");
      c.backend = v;
    } else if (k == "expandable_segments") {
      c.expandable_segments = parse_bool(k, v);
    } else if (k == "release_lock_on_malloc" || k == "release_lock_on_cudamalloc") {
      c.release_lock_on_malloc = parse_bool(k, v);
    } else if (k == "pinned_use_host_register" || k == "pinned_use_cuda_host_register") {
      c.pinned_use_host_register = parse_bool(k, v);
    } else if (k == "pinned_num_register_threads") {
      long long n = std::atoll(v.c_str());
      TORCH_CHECK(n >= 1 && n <= 128 && (n & (n - 1)) == 0,
                  "allocator config: pinned_num_register_threads must be a power of two in [1,128]");
      c.pinned_num_register_threads = (int)n;
    } else if (k == "pinned_use_background_threads") {
      c.pinned_use_background_threads = parse_bool(k, v);
    } else if (k == "cpu") {
      TORCH_CHECK(v == "unified" || v == "default", "allocator config: cpu must be 'unified' or 'default'");
      c.cpu_unified = (v == "unified");
    } else {
      TORCH_CHECK(false, "allocator config: unrecognised key '", k, "'");
    }
  }
  return c;
}

static Config& mutable_config() {
  static Config c = [] {
    Config base;
    if (const char* e = std::getenv("PYTORCH_NO_BLACKWELL_MEMORY_CACHING")) base.no_caching = std::atoi(e) != 0;
    if (const char* e = std::getenv("PYTORCH_BLACKWELL_ALLOC_CONF")) return parse_config(e, base);
    return base;
  }();
  return c;
}
const Config& config() { return mutable_config(); }
void set_config_string(const std::string& s) {
  Config c = parse_config(s, mutable_config());
  TORCH_CHECK(c.backend == mutable_config().backend || !get()->initialized(),
              "allocator backend cannot change after the allocator has been used");
  mutable_config() = c;
}

// ------------------------------------------------------------------ blocks
struct Pool;
struct Block {
  int device = 0;
  cudaStream_t stream = nullptr;  // allocation stream
  std::unordered_set<cudaStream_t> stream_uses;
  size_t size = 0, requested = 0;
  Pool* pool = nullptr;
  void* ptr = nullptr;
  bool allocated = false;
  Block *prev = nullptr, *next = nullptr;
  int event_count = 0;
  int gc_count = 0;
  bool is_split() const { return prev || next; }
};

struct BlockLess {
  bool operator()(const Block* a, const Block* b) const {
    if (a->stream != b->stream) return (uintptr_t)a->stream < (uintptr_t)b->stream;
    if (a->size != b->size) return a->size < b->size;
    return (uintptr_t)a->ptr < (uintptr_t)b->ptr;
  }
};

struct PrivatePool;
struct Pool {
  std::set<Block*, BlockLess> blocks;
  bool is_small;
  PrivatePool* owner = nullptr;
  explicit Pool(bool s, PrivatePool* o = nullptr) : is_small(s), owner(o) {}
};

struct PrivatePool {
  int use_count = 1;
  int live_allocs = 0;
  Pool large{false, this}, small{true, this};
};

struct PoolIdHash {
  size_t operator()(const MempoolId& p) const { return std::hash<uint64_t>()(p.first * 0x9E3779B97F4A7C15ull ^ p.second); }
};

class DeviceAllocatorImpl {
 public:
  DeviceAllocatorImpl(int device, const RawBackend* be) : device_(device), be_(be) {
    stats_.max_split_size = (int64_t)std::min<size_t>(config().max_split_size, (size_t)INT64_MAX);
  }

  static size_t round_size(size_t n) {
    if (n < kMinBlock) return kMinBlock;
    size_t div = config().roundup_power2_divisions;
    if (div > 1 && n > kMinBlock * div) {
      // round up to the next 1/div step between enclosing powers of two
      size_t p2 = (size_t)1 << (63 - __builtin_clzll(n));
      if (p2 == n) return n;
      size_t step = p2 / div;
      if (step >= kMinBlock) return (n + step - 1) / step * step;
    }
    return (n + kMinBlock - 1) / kMinBlock * kMinBlock;
  }

  static size_t segment_size(size_t size) {
    if (size <= kSmallSize) return kSmallBuffer;
    if (size < kMinLargeAlloc) return std::max(config().large_segment_bytes, (size_t)(20u << 20));
    return (size + kRoundLarge - 1) / kRoundLarge * kRoundLarge;
  }

  Block* malloc(size_t orig, cudaStream_t stream) {
    std::unique_lock<std::mutex> lk(mu_);
    process_events();
    size_t size = round_size(orig);
    Pool& pool = pool_for(size, stream);
    Block* b = find_free(pool, size, stream);
    if (!b) {
      if (config().gc_threshold > 0.0) gc_cached();
      b = alloc_segment(pool, size, stream);
      if (!b) {
        ++stats_.num_alloc_retries;
        // first give back only what could satisfy the request, then everything
        if (release_fitting(pool, size)) b = alloc_segment(pool, size, stream);
        if (!b) {
          release_all_cached(/*only_pool=*/nullptr);
          b = alloc_segment(pool, size, stream);
        }
      }
      if (!b) oom(orig, size, lk);
    }
    // split
    if (should_split(b, size)) {
      Block* rem = new Block();
      rem->device = device_;
      rem->stream = b->stream;
      rem->pool = &pool;
      rem->ptr = static_cast<char*>(b->ptr) + size;
      rem->size = b->size - size;
      rem->prev = b;
      rem->next = b->next;
      if (rem->next) rem->next->prev = rem;
      b->next = rem;
      b->size = size;
      pool.blocks.insert(rem);
      bump([&](int t) { stats_.inactive_split[t].inc(1); stats_.inactive_split_bytes[t].inc(rem->size); }, pool);
    }
    b->allocated = true;
    b->requested = orig;
    live_[b->ptr] = b;
    if (pool.owner) ++pool.owner->live_allocs;
    bump([&](int t) {
      stats_.allocation[t].inc(1);
      stats_.allocated_bytes[t].inc(b->size);
      stats_.active[t].inc(1);
      stats_.active_bytes[t].inc(b->size);
      stats_.requested_bytes[t].inc(b->requested);
    }, pool);
    if (b->size >= config().max_split_size) stats_.oversize_allocations.inc(1);
    trace(TraceEntry::ALLOC, b->ptr, b->size, stream);
    return b;
  }

  void free(Block* b) {
    std::lock_guard<std::mutex> lk(mu_);
    b->allocated = false;
    live_.erase(b->ptr);
    Pool& pool = *b->pool;
    bump([&](int t) {
      stats_.allocation[t].dec(1);
      stats_.allocated_bytes[t].dec(b->size);
      stats_.requested_bytes[t].dec(b->requested);
    }, pool);
    if (b->size >= config().max_split_size) stats_.oversize_allocations.dec(1);
    trace(TraceEntry::FREE_REQUESTED, b->ptr, b->size, b->stream);
    if (!b->stream_uses.empty() && be_->device_events) {
      if (capturing_depth_ > 0) {
        // Event queries are illegal while a capture is under way: park the block.
        deferred_.push_back(b);
      } else {
        insert_events(b);
      }
    } else {
      b->stream_uses.clear();
      free_block(b);
    }
  }

  void record_stream(Block* b, cudaStream_t s) {
    std::lock_guard<std::mutex> lk(mu_);
    if (s == b->stream) return;
    b->stream_uses.insert(s);
  }

  Block* find_live(const void* p) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = live_.find(const_cast<void*>(p));
    return it == live_.end() ? nullptr : it->second;
  }

  // Block containing `p` (interior pointers allowed).
  Block* find_containing(const void* p) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = live_.upper_bound(const_cast<void*>(p));
    if (it == live_.begin()) return nullptr;
    --it;
    Block* b = it->second;
    if ((const char*)p < (const char*)b->ptr + b->size) return b;
    return nullptr;
  }

  void empty_cache(MempoolId id) {
    std::lock_guard<std::mutex> lk(mu_);
    if (id.first == 0 && id.second == 0) {
      release_all_cached(nullptr);
    } else {
      auto it = private_.find(id);
      if (it != private_.end()) release_all_cached(it->second.get());
    }
  }

  void set_fraction(double f) {
    std::lock_guard<std::mutex> lk(mu_);
    size_t fr = 0, tot = 0;
    DeviceSwitch sw(be_->device_events ? device_ : -1);
    B200_KERNEL_CALL(be_->mem_info(device_, &fr, &tot));
    fraction_ = f;
    allowed_ = (size_t)(f * (double)tot);
    limited_ = true;
  }
  double fraction() const { return limited_ ? fraction_ : 1.0; }

  DeviceStats stats() {
    std::lock_guard<std::mutex> lk(mu_);
    return stats_;
  }
  void reset_accumulated() {
    std::lock_guard<std::mutex> lk(mu_);
    for_each_stat([](Stat& s) { s.reset_accumulated(); });
    stats_.num_alloc_retries = stats_.num_ooms = stats_.num_sync_all_streams = 0;
    stats_.num_device_alloc = stats_.num_device_free = 0;
  }
  void reset_peak() {
    std::lock_guard<std::mutex> lk(mu_);
    for_each_stat([](Stat& s) { s.reset_peak(); });
  }

  std::vector<SegmentInfo> snapshot(MempoolId filter) {
    std::lock_guard<std::mutex> lk(mu_);
    std::vector<SegmentInfo> out;
    auto visit = [&](Pool& pool, MempoolId id) {
      (void)pool;
      (void)id;
    };
    (void)visit;
    // Every block is either live or in a pool; walk segment heads.
    std::unordered_set<Block*> heads;
    auto add_head = [&](Block* b) {
      while (b->prev) b = b->prev;
      heads.insert(b);
    };
    for (auto& kv : live_) add_head(kv.second);
    auto scan = [&](Pool& p) { for (Block* b : p.blocks) add_head(b); };
    scan(small_);
    scan(large_);
    for (auto& kv : private_) { scan(kv.second->small); scan(kv.second->large); }
    for (Block* b : pending_blocks()) add_head(b);
    for (Block* h : heads) {
      MempoolId id{0, 0};
      if (h->pool->owner) {
        for (auto& kv : private_) if (kv.second.get() == h->pool->owner) id = kv.first;
      }
      if ((filter.first || filter.second) && id != filter) continue;
      SegmentInfo s;
      s.device = device_;
      s.address = (uintptr_t)h->ptr;
      s.stream = h->stream;
      s.is_large = !h->pool->is_small;
      s.is_expandable = false;
      s.pool_id_first = id.first;
      s.pool_id_second = id.second;
      for (Block* b = h; b; b = b->next) {
        s.total_size += b->size;
        BlockInfo bi;
        bi.size = b->size;
        bi.requested = b->requested;
        bi.allocated = b->allocated;
        bi.active = b->allocated || b->event_count > 0 || !b->stream_uses.empty();
        if (bi.allocated) { s.allocated_size += b->size; s.requested_size += b->requested; }
        if (bi.active) s.active_size += b->size;
        s.blocks.push_back(bi);
      }
      out.push_back(std::move(s));
    }
    std::sort(out.begin(), out.end(), [](const SegmentInfo& a, const SegmentInfo& b) { return a.address < b.address; });
    trace(TraceEntry::SNAPSHOT, nullptr, 0, nullptr);
    return out;
  }

  // ------------------------------------------------------- private pools
  void begin_to_pool(MempoolId id, std::function<bool(cudaStream_t)> filter) {
    std::lock_guard<std::mutex> lk(mu_);
    ensure_pool(id);
    captures_.emplace_back(id, std::move(filter));
    ++capturing_depth_;
  }
  void end_to_pool(MempoolId id) {
    std::lock_guard<std::mutex> lk(mu_);
    for (auto it = captures_.begin(); it != captures_.end(); ++it) {
      if (it->first == id) {
        captures_.erase(it);
        --capturing_depth_;
        break;
      }
    }
    if (capturing_depth_ == 0) {
      for (Block* b : deferred_) insert_events(b);
      deferred_.clear();
    }
  }
  void incref_pool(MempoolId id) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = private_.find(id);
    if (it == private_.end()) ensure_pool(id); else ++it->second->use_count;
  }
  void release_pool(MempoolId id) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = private_.find(id);
    if (it == private_.end()) return;
    if (--it->second->use_count <= 0) {
      // Cached blocks return to the device now; the pool object itself goes once no tensor lives in it.
      release_all_cached(it->second.get());
      if (it->second->live_allocs == 0 && it->second->small.blocks.empty() && it->second->large.blocks.empty())
        private_.erase(it);
    }
  }
  int pool_use_count(MempoolId id) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = private_.find(id);
    return it == private_.end() ? 0 : it->second->use_count;
  }

  void set_history(bool on, size_t max_entries) {
    std::lock_guard<std::mutex> lk(mu_);
    history_ = on;
    history_max_ = max_entries ? max_entries : 1;
    if (!on) trace_.clear();
  }
  std::vector<TraceEntry> get_trace() {
    std::lock_guard<std::mutex> lk(mu_);
    return std::vector<TraceEntry>(trace_.begin(), trace_.end());
  }

  std::vector<OomObserver>* observers = nullptr;

 private:
  template <class F>
  void bump(F f, const Pool& pool) {
    f(kAll);
    f(pool.is_small ? kSmall : kLarge);
  }
  template <class F>
  void for_each_stat(F f) {
    for (int t = 0; t < kNumStatTypes; ++t) {
      f(stats_.allocation[t]); f(stats_.segment[t]); f(stats_.active[t]); f(stats_.inactive_split[t]);
      f(stats_.allocated_bytes[t]); f(stats_.reserved_bytes[t]); f(stats_.active_bytes[t]);
      f(stats_.inactive_split_bytes[t]); f(stats_.requested_bytes[t]);
    }
    f(stats_.oversize_allocations);
    f(stats_.oversize_segments);
  }

  void trace(TraceEntry::Action a, void* p, size_t n, cudaStream_t s) {
    if (!history_) return;
    if (trace_.size() >= history_max_) trace_.pop_front();
    trace_.push_back(TraceEntry{a, device_, (uintptr_t)p, n, s, now_ns()});
  }

  PrivatePool* ensure_pool(MempoolId id) {
    auto it = private_.find(id);
    if (it == private_.end()) it = private_.emplace(id, std::make_unique<PrivatePool>()).first;
    return it->second.get();
  }

  Pool& pool_for(size_t size, cudaStream_t stream) {
    if (capturing_depth_ > 0) {
      for (auto& c : captures_) {
        if (c.second(stream)) {
          PrivatePool* pp = ensure_pool(c.first);
          return size <= kSmallSize ? pp->small : pp->large;
        }
      }
    }
    return size <= kSmallSize ? small_ : large_;
  }

  Block* find_free(Pool& pool, size_t size, cudaStream_t stream) {
    Block key;
    key.stream = stream;
    key.size = size;
    key.ptr = nullptr;
    auto it = pool.blocks.lower_bound(&key);
    if (it == pool.blocks.end() || (*it)->stream != stream) return nullptr;
    Block* b = *it;
    size_t msz = config().max_split_size;
    // An oversize block is only handed out whole, and only for an oversize request that nearly fills it.
    if (size < msz && b->size >= msz) return nullptr;
    if (size >= msz && b->size >= size + kMinLargeAlloc * 2) return nullptr;
    pool.blocks.erase(it);
    if (b->is_split()) {
      bump([&](int t) { stats_.inactive_split[t].dec(1); stats_.inactive_split_bytes[t].dec(b->size); }, pool);
    }
    b->gc_count = 0;
    return b;
  }

  bool should_split(const Block* b, size_t size) const {
    size_t rem = b->size - size;
    if (b->pool->is_small) return rem >= kMinBlock;
    if (config().max_split_size != SIZE_MAX) return size < config().max_split_size && rem > kSmallSize;
    // default policy: huge tail remainders on a 180 GB part are fine to keep, but tiny ones are not worth a node
    (void)kHugeNoSplit;
    return rem > kSmallSize;
  }

  Block* alloc_segment(Pool& pool, size_t size, cudaStream_t stream) {
    size_t seg = segment_size(size);
    if (limited_ && (size_t)stats_.reserved_bytes[kAll].current + seg > allowed_) return nullptr;
    void* p = nullptr;
    int e;
    {
      DeviceSwitch sw(be_->device_events ? device_ : -1);
      if (capturing_depth_ > 0 && be_->device_events) {
        // A driver allocation is not a captured operation: step out of the capture's error mode for it.
        cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
        cudaThreadExchangeStreamCaptureMode(&mode);
        e = be_->raw_alloc(&p, seg, device_, stream);
        cudaThreadExchangeStreamCaptureMode(&mode);
      } else {
        e = be_->raw_alloc(&p, seg, device_, stream);
      }
    }
    if (e != 0) {
      if (be_->device_events) (void)cudaGetLastError();
      if (e != (int)cudaErrorMemoryAllocation) check_cuda((cudaError_t)e, "raw_alloc", __FILE__, __LINE__);
      return nullptr;
    }
    ++stats_.num_device_alloc;
    Block* b = new Block();
    b->device = device_;
    b->stream = stream;
    b->size = seg;
    b->pool = &pool;
    b->ptr = p;
    bump([&](int t) { stats_.segment[t].inc(1); stats_.reserved_bytes[t].inc(seg); }, pool);
    if (seg >= config().max_split_size) stats_.oversize_segments.inc(1);
    trace(TraceEntry::SEGMENT_ALLOC, p, seg, stream);
    return b;
  }

  void release_block(Block* b) {
    // b is a whole, free segment sitting in its pool
    Pool& pool = *b->pool;
    {
      DeviceSwitch sw(be_->device_events ? device_ : -1);
      B200_KERNEL_CALL(be_->raw_free(b->ptr, b->size, device_, b->stream));
    }
    ++stats_.num_device_free;
    bump([&](int t) { stats_.segment[t].dec(1); stats_.reserved_bytes[t].dec(b->size); }, pool);
    if (b->size >= config().max_split_size) stats_.oversize_segments.dec(1);
    trace(TraceEntry::SEGMENT_FREE, b->ptr, b->size, b->stream);
    pool.blocks.erase(b);
    delete b;
  }

  bool release_fitting(Pool& pool, size_t size) {
    // Only worth it for oversize requests: free the smallest whole cached segment >= size.
    if (config().max_split_size == SIZE_MAX || size < config().max_split_size) return false;
    for (Block* b : pool.blocks) {
      if (!b->is_split() && b->size >= size) {
        sync_and_drain();
        release_block(b);
        return true;
      }
    }
    return false;
  }

  void release_pool_blocks(Pool& pool) {
    std::vector<Block*> whole;
    for (Block* b : pool.blocks) if (!b->is_split()) whole.push_back(b);
    for (Block* b : whole) release_block(b);
  }

  void sync_and_drain() {
    // Wait for every outstanding cross-stream use so those blocks become releasable.
    if (be_->device_events && capturing_depth_ == 0) {
      for (auto& q : events_) {
        for (auto& eb : q.second) {
          B200_CUDA_CHECK(cudaEventSynchronize(eb.first));
          return_event(eb.first);
          Block* b = eb.second;
          if (--b->event_count == 0) free_block(b);
        }
      }
      events_.clear();
      ++stats_.num_sync_all_streams;
    }
  }

  void release_all_cached(PrivatePool* only) {
    sync_and_drain();
    if (only) {
      release_pool_blocks(only->small);
      release_pool_blocks(only->large);
      return;
    }
    release_pool_blocks(small_);
    release_pool_blocks(large_);
    for (auto it = private_.begin(); it != private_.end();) {
      PrivatePool* pp = it->second.get();
      if (pp->use_count <= 0) {
        release_pool_blocks(pp->small);
        release_pool_blocks(pp->large);
        if (pp->live_allocs == 0 && pp->small.blocks.empty() && pp->large.blocks.empty()) {
          it = private_.erase(it);
          continue;
        }
      }
      ++it;
    }
  }

  void gc_cached() {
    size_t tot_allowed = allowed_;
    if (!limited_) {
      size_t fr = 0, tot = 0;
      DeviceSwitch sw(be_->device_events ? device_ : -1);
      if (be_->mem_info(device_, &fr, &tot) != 0) return;
      tot_allowed = tot;
    }
    size_t target = (size_t)(config().gc_threshold * (double)tot_allowed);
    if ((size_t)stats_.reserved_bytes[kAll].current <= target) return;
    size_t excess = (size_t)stats_.reserved_bytes[kAll].current - target;
    // age the cached whole large segments; free the oldest until under target
    std::vector<Block*> cands;
    for (Block* b : large_.blocks) if (!b->is_split()) { ++b->gc_count; cands.push_back(b); }
    std::sort(cands.begin(), cands.end(), [](Block* a, Block* b) { return a->gc_count > b->gc_count; });
    size_t freed = 0;
    for (Block* b : cands) {
      if (freed >= excess) break;
      freed += b->size;
      release_block(b);
    }
  }

  [[noreturn]] void oom(size_t orig, size_t size, std::unique_lock<std::mutex>& lk) {
    ++stats_.num_ooms;
    size_t fr = 0, tot = 0;
    {
      DeviceSwitch sw(be_->device_events ? device_ : -1);
      be_->mem_info(device_, &fr, &tot);
    }
    trace(TraceEntry::OOM, nullptr, size, nullptr);
    DeviceStats s = stats_;
    lk.unlock();
    if (observers) for (auto& o : *observers) o(device_, orig, tot, fr);
    auto mib = [](int64_t b) { return std::to_string(b >> 20) + " MiB"; };
    std::string lim = limited_ ? (" Process memory fraction limits this device to " + mib((int64_t)allowed_) + ".") : "";
    TORCH_CHECK_WITH(OutOfMemoryError, false, "blackwell out of memory. Tried to allocate ", mib((int64_t)size),
                     " on device ", device_, " (", mib((int64_t)tot), " total, ", mib((int64_t)fr), " free; ",
                     mib(s.allocated_bytes[kAll].current), " allocated by tensors, ",
                     mib(s.reserved_bytes[kAll].current), " reserved by the caching allocator).", lim,
                     " If reserved >> allocated, try PYTORCH_BLACKWELL_ALLOC_CONF=max_split_size_mb:<n> or "
                     "garbage_collection_threshold:<f> to reduce fragmentation.");
  }

  void free_block(Block* b) {
    Pool& pool = *b->pool;
    size_t orig_size = b->size;
    bool was_split_inactive_delta = false;
    (void)was_split_inactive_delta;
    trace(TraceEntry::FREE_COMPLETED, b->ptr, b->size, b->stream);
    bump([&](int t) { stats_.active[t].dec(1); stats_.active_bytes[t].dec(orig_size); }, pool);
    if (pool.owner) --pool.owner->live_allocs;
    int64_t net_inactive_blocks = 0, net_inactive_bytes = 0;
    for (Block* nb : {b->prev, b->next}) {
      if (!nb || nb->allocated || nb->event_count > 0 || !nb->stream_uses.empty()) continue;
      if (!pool.blocks.count(nb)) continue;  // parked (deferred) blocks are not mergeable
      // merge nb into b
      pool.blocks.erase(nb);
      net_inactive_blocks -= 1;
      net_inactive_bytes -= (int64_t)nb->size;
      if (nb == b->prev) {
        b->ptr = nb->ptr;
        b->prev = nb->prev;
        if (b->prev) b->prev->next = b;
      } else {
        b->next = nb->next;
        if (b->next) b->next->prev = b;
      }
      b->size += nb->size;
      delete nb;
    }
    pool.blocks.insert(b);
    if (b->is_split()) {
      net_inactive_blocks += 1;
      net_inactive_bytes += (int64_t)b->size;
    }
    bump([&](int t) {
      if (net_inactive_blocks > 0) stats_.inactive_split[t].inc(net_inactive_blocks);
      else if (net_inactive_blocks < 0) stats_.inactive_split[t].dec(-net_inactive_blocks);
      if (net_inactive_bytes > 0) stats_.inactive_split_bytes[t].inc(net_inactive_bytes);
      else if (net_inactive_bytes < 0) stats_.inactive_split_bytes[t].dec(-net_inactive_bytes);
    }, pool);
    if (pool.owner && pool.owner->use_count <= 0 && pool.owner->live_allocs == 0) {
      // last tensor of a released pool: give the memory back
      release_pool_blocks(pool.owner->small);
      release_pool_blocks(pool.owner->large);
    }
  }

  cudaEvent_t get_event() {
    if (!event_pool_.empty()) {
      cudaEvent_t e = event_pool_.back();
      event_pool_.pop_back();
      return e;
    }
    cudaEvent_t e;
    B200_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    return e;
  }
  void return_event(cudaEvent_t e) { event_pool_.push_back(e); }

  void insert_events(Block* b) {
    DeviceSwitch sw(device_);
    std::unordered_set<cudaStream_t> uses;
    uses.swap(b->stream_uses);
    for (cudaStream_t s : uses) {
      cudaEvent_t e = get_event();
      B200_CUDA_CHECK(cudaEventRecord(e, s));
      ++b->event_count;
      events_[s].emplace_back(e, b);
    }
  }

  void process_events() {
    if (events_.empty() || capturing_depth_ > 0) return;
    for (auto it = events_.begin(); it != events_.end();) {
      auto& q = it->second;
      while (!q.empty()) {
        cudaEvent_t e = q.front().first;
        cudaError_t r = cudaEventQuery(e);
        if (r == cudaErrorNotReady) {
          (void)cudaGetLastError();
          break;
        }
        B200_CUDA_CHECK(r);
        return_event(e);
        Block* b = q.front().second;
        q.pop_front();
        if (--b->event_count == 0) free_block(b);
      }
      if (q.empty()) it = events_.erase(it); else ++it;
    }
  }

  std::vector<Block*> pending_blocks() {
    std::vector<Block*> v;
    for (auto& q : events_) for (auto& eb : q.second) v.push_back(eb.second);
    for (Block* b : deferred_) v.push_back(b);
    return v;
  }

  int device_;
  const RawBackend* be_;
  std::mutex mu_;
  Pool small_{true}, large_{false};
  std::map<void*, Block*> live_;
  std::unordered_map<MempoolId, std::unique_ptr<PrivatePool>, PoolIdHash> private_;
  std::vector<std::pair<MempoolId, std::function<bool(cudaStream_t)>>> captures_;
  int capturing_depth_ = 0;
  std::vector<Block*> deferred_;
  std::unordered_map<cudaStream_t, std::deque<std::pair<cudaEvent_t, Block*>>> events_;
  std::vector<cudaEvent_t> event_pool_;
  DeviceStats stats_;
  bool limited_ = false;
  double fraction_ = 1.0;
  size_t allowed_ = 0;
  bool history_ = false;
  size_t history_max_ = 1;
  std::deque<TraceEntry> trace_;
};

// ------------------------------------------------------------------ facade
namespace {
std::vector<OomObserver> g_observers;
std::mutex g_nocache_mu;
struct NoCacheEntry { size_t size; int device; CachingAllocator* owner; };
std::unordered_map<void*, NoCacheEntry> g_nocache;

void deleter(void* ctx);
}  // namespace

CachingAllocator::CachingAllocator(const RawBackend* backend, int num_devices) : backend_(backend) {
  if (num_devices > 0) init(num_devices);
}
CachingAllocator::~CachingAllocator() = default;

void CachingAllocator::init(int n) {
  static std::mutex mu;
  std::lock_guard<std::mutex> g(mu);
  while ((int)devs_.size() < n) {
    devs_.emplace_back(std::make_unique<DeviceAllocatorImpl>((int)devs_.size(), backend_));
    devs_.back()->observers = &g_observers;
  }
}

namespace {
struct Ctx {
  CachingAllocator* owner;
  Block* block;     // null in no-caching mode
  void* ptr;
};
// ctx pointers are Block* tagged through a side table to keep DataPtr contexts one word.
std::mutex g_ctx_mu;
std::unordered_map<void*, CachingAllocator*> g_block_owner;  // Block* -> owner

void deleter(void* ctx) {
  Block* b = static_cast<Block*>(ctx);
  CachingAllocator* owner;
  {
    std::lock_guard<std::mutex> g(g_ctx_mu);
    auto it = g_block_owner.find(ctx);
    TORCH_INTERNAL_ASSERT(it != g_block_owner.end(), "blackwell allocator: freeing an unknown block");
    owner = it->second;
    g_block_owner.erase(it);
  }
  owner->raw_delete(b->ptr);
}

void nocache_deleter(void* p) {
  NoCacheEntry e;
  {
    std::lock_guard<std::mutex> g(g_nocache_mu);
    auto it = g_nocache.find(p);
    if (it == g_nocache.end()) return;
    e = it->second;
    g_nocache.erase(it);
  }
  DeviceSwitch sw(e.owner->backend()->device_events ? e.device : -1);
  B200_CUDA_WARN((cudaError_t)e.owner->backend()->raw_free(p, e.size, e.device, nullptr));
}
}  // namespace

c10::DataPtr CachingAllocator::allocate(size_t n) {
  int device = 0;
  cudaStream_t stream = nullptr;
  if (backend_->device_events) {
    device = current_device();
    stream = get_current_stream(device).stream();
  }
  if ((int)devs_.size() <= device) init(std::max<int>(device + 1, backend_->device_events ? device_count() : 1));
  if (n == 0) return c10::DataPtr(nullptr, nullptr, &c10::detail::deleteNothing, make_device(device));
  if (config().no_caching || backend_ == &g_plug) {
    // Pass-through: user plug-ins and the no-caching debug mode see every allocation and free.
    void* p = nullptr;
    int e = backend_->raw_alloc(&p, n, device, stream);
    if (e != 0) check_cuda((cudaError_t)e, "raw_alloc (no caching)", __FILE__, __LINE__);
    {
      std::lock_guard<std::mutex> g(g_nocache_mu);
      g_nocache[p] = NoCacheEntry{n, device, this};
    }
    return c10::DataPtr(p, p, &nocache_deleter, make_device(device));
  }
  Block* b = devs_[device]->malloc(n, stream);
  {
    std::lock_guard<std::mutex> g(g_ctx_mu);
    g_block_owner[b] = this;
  }
  return c10::DataPtr(b->ptr, b, &deleter, make_device(device));
}

c10::DeleterFnPtr CachingAllocator::raw_deleter() const { return &deleter; }

void CachingAllocator::copy_data(void* dst, const void* src, size_t n) const {
  if (backend_->device_events) {
    B200_CUDA_CHECK(cudaMemcpy(dst, src, n, cudaMemcpyDeviceToDevice));
  } else {
    std::memcpy(dst, src, n);
  }
}

void* CachingAllocator::raw_alloc(size_t n, int device, cudaStream_t stream) {
  if (n == 0) return nullptr;
  if ((int)devs_.size() <= device) init(device + 1);
  return devs_[device]->malloc(n, stream)->ptr;
}

void CachingAllocator::raw_delete(void* p) {
  if (!p) return;
  for (auto& d : devs_) {
    if (Block* b = d->find_live(p)) {
      d->free(b);
      return;
    }
  }
  TORCH_CHECK(false, "blackwell allocator: pointer ", p, " is not a live allocation");
}

void CachingAllocator::record_stream(const c10::DataPtr& p, int device, cudaStream_t stream) {
  if (!p.get()) return;
  if (p.get_deleter() != &deleter) return;  // foreign / no-cache memory: nothing to track
  Block* b = static_cast<Block*>(p.get_context());
  devs_[b->device]->record_stream(b, stream);
}

void CachingAllocator::record_stream_ptr(void* p, int device, cudaStream_t stream) {
  if (!p || device >= (int)devs_.size()) return;
  if (Block* b = devs_[device]->find_containing(p)) devs_[device]->record_stream(b, stream);
}

void CachingAllocator::empty_cache(int device, MempoolId pool) {
  for (int d = 0; d < (int)devs_.size(); ++d)
    if (device < 0 || d == device) devs_[d]->empty_cache(pool);
}

void CachingAllocator::set_memory_fraction(double f, int device) {
  TORCH_CHECK(f >= 0.0 && f <= 1.0, "invalid memory fraction ", f, " (must be in [0,1])");
  if ((int)devs_.size() <= device) init(device + 1);
  devs_[device]->set_fraction(f);
}
double CachingAllocator::get_memory_fraction(int device) {
  if ((int)devs_.size() <= device) return 1.0;
  return devs_[device]->fraction();
}

DeviceStats CachingAllocator::stats(int device) {
  if ((int)devs_.size() <= device) init(device + 1);
  return devs_[device]->stats();
}
void CachingAllocator::reset_accumulated_stats(int device) {
  if ((int)devs_.size() > device) devs_[device]->reset_accumulated();
}
void CachingAllocator::reset_peak_stats(int device) {
  if ((int)devs_.size() > device) devs_[device]->reset_peak();
}

std::vector<SegmentInfo> CachingAllocator::snapshot(int device, MempoolId pool) {
  std::vector<SegmentInfo> out;
  for (int d = 0; d < (int)devs_.size(); ++d) {
    if (device >= 0 && d != device) continue;
    auto v = devs_[d]->snapshot(pool);
    out.insert(out.end(), v.begin(), v.end());
  }
  return out;
}

void* CachingAllocator::base_allocation(void* p, size_t* size) {
  for (auto& d : devs_) {
    if (Block* b = d->find_containing(p)) {
      Block* h = b;
      while (h->prev) h = h->prev;
      size_t tot = 0;
      for (Block* x = h; x; x = x->next) tot += x->size;
      if (size) *size = tot;
      return h->ptr;
    }
  }
  TORCH_CHECK(false, "blackwell allocator: pointer ", p, " does not belong to a live allocation");
}

void CachingAllocator::mem_info(int device, size_t* f, size_t* t) {
  DeviceSwitch sw(backend_->device_events ? device : -1);
  B200_KERNEL_CALL(backend_->mem_info(device, f, t));
}

bool CachingAllocator::owns(const void* p, int* device) {
  for (int d = 0; d < (int)devs_.size(); ++d) {
    if (devs_[d]->find_containing(p)) {
      if (device) *device = d;
      return true;
    }
  }
  return false;
}

void CachingAllocator::begin_allocate_to_pool(int device, MempoolId pool, std::function<bool(cudaStream_t)> filter) {
  if ((int)devs_.size() <= device) init(device + 1);
  devs_[device]->begin_to_pool(pool, std::move(filter));
}
void CachingAllocator::end_allocate_to_pool(int device, MempoolId pool) { devs_[device]->end_to_pool(pool); }
void CachingAllocator::release_pool(int device, MempoolId pool) {
  if ((int)devs_.size() > device) devs_[device]->release_pool(pool);
}
void CachingAllocator::create_or_incref_pool(int device, MempoolId pool) {
  if ((int)devs_.size() <= device) init(device + 1);
  devs_[device]->incref_pool(pool);
}
int CachingAllocator::pool_use_count(int device, MempoolId pool) {
  if ((int)devs_.size() <= device) return 0;
  return devs_[device]->pool_use_count(pool);
}

void CachingAllocator::attach_oom_observer(OomObserver o) { g_observers.push_back(std::move(o)); }
void CachingAllocator::record_history(bool enabled, size_t max_entries) {
  for (auto& d : devs_) d->set_history(enabled, max_entries);
}
std::vector<TraceEntry> CachingAllocator::trace(int device) {
  if ((int)devs_.size() <= device) return {};
  return devs_[device]->get_trace();
}

MempoolId CachingAllocator::new_pool_id(bool user_created) {
  // ids handed to graph capture use the second slot, user MemPools the first: the two sequences never collide
  static std::atomic<uint64_t> uid{1}, gid{1};
  if (user_created) return {uid.fetch_add(1), 0};
  return {0, gid.fetch_add(1)};
}

// ---------------------------------------------------------------- selection
namespace {
CachingAllocator* g_current = nullptr;
std::mutex g_sel_mu;
}  // namespace

CachingAllocator* get() {
  if (C10_LIKELY(g_current != nullptr)) return g_current;
  std::lock_guard<std::mutex> g(g_sel_mu);
  if (!g_current) {
    const std::string& b = config().backend;
    const RawBackend* be = b == "unified" ? unified_backend()
                           : b == "cudaMallocAsync" ? async_backend()
                           : b == "host" ? host_backend()
                                         : native_backend();
    g_current = new CachingAllocator(be);  // leaked on purpose: tensors may outlive static destruction
  }
  return g_current;
}

void install_pluggable(int (*malloc_fn)(void**, size_t, int, cudaStream_t),
                       int (*free_fn)(void*, size_t, int, cudaStream_t)) {
  std::lock_guard<std::mutex> g(g_sel_mu);
  TORCH_CHECK(!g_current || !g_current->initialized(),
              "Can't swap an already initialized allocator: change_current_allocator must run before the first "
              "blackwell allocation");
  g_plug.raw_alloc = malloc_fn;
  g_plug.raw_free = free_fn;
  g_current = new CachingAllocator(&g_plug);
}

std::string backend_name() { return get()->backend()->name; }

}  // namespace alloc
}  // namespace b200
