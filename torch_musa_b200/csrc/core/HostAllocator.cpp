#include "core/HostAllocator.h"

#include "core/CachingAllocator.h"

#include <c10/core/CPUAllocator.h>

#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

namespace b200 {
namespace host {

namespace {

struct HBlock {
  void* ptr = nullptr;
  size_t size = 0;       // bucket size
  bool registered = false;  // malloc + cudaHostRegister instead of cudaHostAlloc
  bool allocated = false;
  int pending = 0;
  std::vector<std::pair<int, cudaStream_t>> uses;  // (device, stream) recorded since allocation
};

size_t bucket(size_t n) {
  if (n <= 64) return 64;
  size_t p = (size_t)1 << (64 - __builtin_clzll(n - 1));
  return p;
}

class PinnedAllocator final : public c10::Allocator {
 public:
  c10::DataPtr allocate(size_t n) override {
    if (n == 0) return c10::DataPtr(nullptr, nullptr, &c10::detail::deleteNothing, c10::Device(c10::kCPU));
    HBlock* b = get_block(n);
    return c10::DataPtr(b->ptr, b, &PinnedAllocator::deleter, c10::Device(c10::kCPU));
  }
  c10::DeleterFnPtr raw_deleter() const override { return &PinnedAllocator::deleter; }
  void copy_data(void* dst, const void* src, size_t n) const override { std::memcpy(dst, src, n); }

  static void deleter(void* ctx);

  HBlock* get_block(size_t n) {
    size_t sz = bucket(n);
    {
      std::lock_guard<std::mutex> g(mu_);
      process_events();
      auto& fl = free_[sz];
      if (!fl.empty()) {
        HBlock* b = fl.back();
        fl.pop_back();
        b->allocated = true;
        ++st_.allocations; ++st_.reuse_hits;
        --st_.cached_blocks; st_.cached_bytes -= (int64_t)sz;
        ++st_.active_blocks; st_.active_bytes += (int64_t)sz;
        return b;
      }
    }
    auto* b = new HBlock();
    b->size = sz;
    const auto& cfg = alloc::config();
    if (cfg.pinned_use_host_register) {
      void* p = nullptr;
      TORCH_CHECK(posix_memalign(&p, 4096, sz) == 0, "pinned allocator: host malloc of ", sz, " bytes failed");
      prefault(p, sz, cfg.pinned_num_register_threads);
      B200_CUDA_CHECK(cudaHostRegister(p, sz, cudaHostRegisterDefault));
      b->ptr = p;
      b->registered = true;
    } else {
      B200_CUDA_CHECK(cudaHostAlloc(&b->ptr, sz, cudaHostAllocDefault));
    }
    b->allocated = true;
    std::lock_guard<std::mutex> g(mu_);
    blocks_[b->ptr] = b;
    ++st_.allocations; ++st_.device_allocs; ++st_.active_blocks; st_.active_bytes += (int64_t)sz;
    return b;
  }

  static void prefault(void* p, size_t n, int threads) {
    // Touch every page so cudaHostRegister does not pay for the faults serially.
    auto touch = [](char* b, char* e) { for (; b < e; b += 4096) *b = 0; };
    char* c = static_cast<char*>(p);
    if (threads <= 1 || n < ((size_t)64 << 20)) { touch(c, c + n); return; }
    std::vector<std::thread> ts;
    size_t per = ((n / threads) + 4095) / 4096 * 4096;
    for (int i = 0; i < threads; ++i) {
      char* b = c + per * i;
      if (b >= c + n) break;
      char* e = std::min(b + per, c + n);
      ts.emplace_back(touch, b, e);
    }
    for (auto& t : ts) t.join();
  }

  void free_block(HBlock* b) {
    std::lock_guard<std::mutex> g(mu_);
    ++st_.frees;
    --st_.active_blocks; st_.active_bytes -= (int64_t)b->size;
    b->allocated = false;
    if (b->uses.empty()) {
      to_cache(b);
      return;
    }
    for (auto& u : b->uses) {
      DeviceSwitch sw(u.first);
      cudaEvent_t e = get_event(u.first);
      B200_CUDA_CHECK(cudaEventRecord(e, u.second));
      ++b->pending;
      ++st_.events_pending;
      events_.push_back({e, u.first, b});
    }
    b->uses.clear();
  }

  bool record(const void* p, void* ctx, const Stream& s) {
    std::lock_guard<std::mutex> g(mu_);
    HBlock* b = nullptr;
    if (ctx) {
      auto it = blocks_.find(static_cast<HBlock*>(ctx)->ptr);
      // ctx is only trusted when it is one of our block records
      if (it != blocks_.end() && it->second == ctx) b = it->second;
    }
    if (!b) b = find_containing(p);
    if (!b) return false;
    auto key = std::make_pair((int)s.device_index(), s.stream());
    for (auto& u : b->uses) if (u == key) return true;
    b->uses.push_back(key);
    return true;
  }

  bool contains(const void* p) {
    std::lock_guard<std::mutex> g(mu_);
    return find_containing(p) != nullptr;
  }

  void empty() {
    std::lock_guard<std::mutex> g(mu_);
    // wait for pending events first
    for (auto& e : events_) {
      B200_CUDA_CHECK(cudaEventSynchronize(e.ev));
      put_event(e.device, e.ev);
      --st_.events_pending;
      if (--e.block->pending == 0 && !e.block->allocated) to_cache(e.block);
    }
    events_.clear();
    for (auto& kv : free_) {
      for (HBlock* b : kv.second) {
        blocks_.erase(b->ptr);
        if (b->registered) {
          B200_CUDA_WARN(cudaHostUnregister(b->ptr));
          std::free(b->ptr);
        } else {
          B200_CUDA_WARN(cudaFreeHost(b->ptr));
        }
        --st_.cached_blocks; st_.cached_bytes -= (int64_t)b->size;
        delete b;
      }
      kv.second.clear();
    }
  }

  HostStats stats() {
    std::lock_guard<std::mutex> g(mu_);
    return st_;
  }

 private:
  struct Ev { cudaEvent_t ev; int device; HBlock* block; };

  HBlock* find_containing(const void* p) {
    auto it = blocks_.upper_bound(const_cast<void*>(p));
    if (it == blocks_.begin()) return nullptr;
    --it;
    HBlock* b = it->second;
    return ((const char*)p < (const char*)b->ptr + b->size) ? b : nullptr;
  }
  void to_cache(HBlock* b) {
    free_[b->size].push_back(b);
    ++st_.cached_blocks; st_.cached_bytes += (int64_t)b->size;
  }
  cudaEvent_t get_event(int dev) {
    auto& pool = ev_pool_[dev];
    if (!pool.empty()) { auto e = pool.back(); pool.pop_back(); return e; }
    cudaEvent_t e;
    B200_CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    return e;
  }
  void put_event(int dev, cudaEvent_t e) { ev_pool_[dev].push_back(e); }
  void process_events() {
    while (!events_.empty()) {
      Ev& e = events_.front();
      cudaError_t r = cudaEventQuery(e.ev);
      if (r == cudaErrorNotReady) { (void)cudaGetLastError(); break; }
      B200_CUDA_CHECK(r);
      put_event(e.device, e.ev);
      --st_.events_pending;
      if (--e.block->pending == 0 && !e.block->allocated) to_cache(e.block);
      events_.pop_front();
    }
  }

  std::mutex mu_;
  std::map<void*, HBlock*> blocks_;
  std::unordered_map<size_t, std::vector<HBlock*>> free_;
  std::deque<Ev> events_;
  std::unordered_map<int, std::vector<cudaEvent_t>> ev_pool_;
  HostStats st_;
};

PinnedAllocator* pinned() {
  static PinnedAllocator* a = new PinnedAllocator();  // outlives static destruction
  return a;
}

void PinnedAllocator::deleter(void* ctx) { pinned()->free_block(static_cast<HBlock*>(ctx)); }

// ----------------------------------------------------------- managed CPU
std::mutex g_managed_mu;
std::map<const void*, size_t> g_managed;

void managed_deleter(void* p) {
  {
    std::lock_guard<std::mutex> g(g_managed_mu);
    g_managed.erase(p);
  }
  B200_CUDA_WARN(cudaFree(p));
}

class UnifiedCPUAllocator final : public c10::Allocator {
 public:
  c10::DataPtr allocate(size_t n) override {
    if (n == 0) return c10::DataPtr(nullptr, nullptr, &c10::detail::deleteNothing, c10::Device(c10::kCPU));
    void* p = nullptr;
    B200_CUDA_CHECK(cudaMallocManaged(&p, n, cudaMemAttachGlobal));
    {
      std::lock_guard<std::mutex> g(g_managed_mu);
      g_managed[p] = n;
    }
    return c10::DataPtr(p, p, &managed_deleter, c10::Device(c10::kCPU));
  }
  c10::DeleterFnPtr raw_deleter() const override { return &managed_deleter; }
  void copy_data(void* dst, const void* src, size_t n) const override { std::memcpy(dst, src, n); }
};

c10::Allocator* g_prev_cpu = nullptr;
bool g_unified_on = false;

}  // namespace

c10::Allocator* pinned_allocator() { return pinned(); }
bool record_event(const void* ptr, void* ctx, const Stream& stream) { return pinned()->record(ptr, ctx, stream); }
bool is_pinned(const void* ptr) {
  if (!ptr) return false;
  if (pinned()->contains(ptr)) return true;
  if (device_count() == 0) return false;
  cudaPointerAttributes attr{};
  cudaError_t e = cudaPointerGetAttributes(&attr, ptr);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return false; }
  return attr.type == cudaMemoryTypeHost;
}
void empty_cache() { pinned()->empty(); }
HostStats stats() { return pinned()->stats(); }

c10::Allocator* unified_cpu_allocator() {
  static UnifiedCPUAllocator* a = new UnifiedCPUAllocator();
  return a;
}

void set_unified_cpu_allocator(bool on) {
  std::lock_guard<std::mutex> g(g_managed_mu);
  if (on == g_unified_on) return;
  if (on) {
    g_prev_cpu = c10::GetAllocator(c10::kCPU);
    c10::SetAllocator(c10::kCPU, unified_cpu_allocator(), /*priority=*/255);
  } else {
    c10::SetAllocator(c10::kCPU, g_prev_cpu ? g_prev_cpu : c10::GetDefaultCPUAllocator(), /*priority=*/255);
  }
  g_unified_on = on;
}
bool unified_cpu_allocator_enabled() { return g_unified_on; }

bool is_managed_ptr(const void* p) {
  std::lock_guard<std::mutex> g(g_managed_mu);
  auto it = g_managed.upper_bound(p);
  if (it == g_managed.begin()) return false;
  --it;
  return (const char*)p < (const char*)it->first + it->second;
}

}  // namespace host
}  // namespace b200
