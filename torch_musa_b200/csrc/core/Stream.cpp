#include "core/Stream.h"
#include <cstdlib>
#include <vector>
#include <map>

#include <c10/util/CallOnce.h>

#include <array>
#include <atomic>
#include <mutex>

namespace b200 {

namespace {

struct DevicePool {
  c10::once_flag once;
  cudaStream_t streams[kMaxPriorities][kStreamsPerPool]{};
  std::atomic<uint32_t> next[kMaxPriorities]{};
};

std::array<DevicePool, kMaxDevices> g_pools;
int g_num_prio = -1;
int g_least = 0, g_greatest = 0;
c10::once_flag g_prio_once;

void init_priorities() {
  c10::call_once(g_prio_once, [] {
    int least = 0, greatest = 0;
    B200_CUDA_CHECK(cudaDeviceGetStreamPriorityRange(&least, &greatest));
    g_least = least;
    g_greatest = greatest;
    int n = least - greatest + 1;  // greatest is numerically the smallest
    g_num_prio = n < 1 ? 1 : (n > kMaxPriorities ? kMaxPriorities : n);
  });
}

void init_pool(c10::DeviceIndex d) {
  init_priorities();
  c10::call_once(g_pools[d].once, [d] {
    DeviceSwitch sw(d);
    for (int p = 0; p < g_num_prio; ++p) {
      for (int i = 0; i < kStreamsPerPool; ++i) {
        // slot p holds CUDA priority (least - p): p == 0 is the default priority.
        B200_CUDA_CHECK(cudaStreamCreateWithPriority(&g_pools[d].streams[p][i], cudaStreamNonBlocking, g_least - p));
      }
    }
  });
}

inline c10::DeviceIndex resolve(c10::DeviceIndex d) {
  if (d < 0) d = current_device();
  TORCH_CHECK(d < device_count(), "invalid blackwell device index ", (int)d);
  return d;
}

inline c10::Stream make(c10::DeviceIndex d, c10::StreamId id) {
  return c10::Stream(c10::Stream::UNSAFE, make_device(d), id);
}

// thread-local current stream ids, one per device; 0 == default stream
thread_local std::array<c10::StreamId, kMaxDevices> tl_current{};

}  // namespace

int num_priorities() {
  init_priorities();
  return g_num_prio;
}

void priority_range(int* least, int* greatest) {
  init_priorities();
  // Reported torch-style: 0 is the default, the most urgent level is -(n-1).
  *least = 0;
  *greatest = -(g_num_prio - 1);
}

cudaStream_t stream_from_c10(c10::Stream s) {
  TORCH_CHECK(s.device_type() == kDeviceType, "expected a blackwell stream, got ", s);
  c10::StreamId id = s.id();
  if (id == 0) return nullptr;  // legacy default stream
  if (id & 1) {
    uint64_t v = static_cast<uint64_t>(id) >> 1;
    int p = static_cast<int>(v / kStreamsPerPool), i = static_cast<int>(v % kStreamsPerPool);
    TORCH_CHECK(p < kMaxPriorities, "corrupt blackwell stream id ", id);
    init_pool(s.device_index());
    return g_pools[s.device_index()].streams[p][i];
  }
  return reinterpret_cast<cudaStream_t>(static_cast<uintptr_t>(id));
}

cudaStream_t Stream::stream() const { return stream_from_c10(s_); }

bool Stream::query() const {
  DeviceSwitch sw(device_index());
  cudaError_t e = cudaStreamQuery(stream());
  if (e == cudaSuccess) return true;
  if (e != cudaErrorNotReady) B200_CUDA_CHECK(e);
  (void)cudaGetLastError();
  return false;
}

void Stream::synchronize() const {
  DeviceSwitch sw(device_index());
  note_implicit_sync("Stream::synchronize");
  B200_CUDA_CHECK(cudaStreamSynchronize(stream()));
}

int Stream::priority() const {
  c10::StreamId id = s_.id();
  if (id & 1) return -static_cast<int>((static_cast<uint64_t>(id) >> 1) / kStreamsPerPool);
  if (id == 0) return 0;
  DeviceSwitch sw(device_index());
  int p = 0;
  B200_CUDA_CHECK(cudaStreamGetPriority(stream(), &p));
  init_priorities();
  return p - g_least;  // 0 for default, negative for urgent
}

Stream get_stream_from_pool(int priority, c10::DeviceIndex device) {
  device = resolve(device);
  init_pool(device);
  int p = priority >= 0 ? 0 : -priority;
  if (p > g_num_prio - 1) p = g_num_prio - 1;
  uint32_t i = g_pools[device].next[p].fetch_add(1, std::memory_order_relaxed) % kStreamsPerPool;
  c10::StreamId id = static_cast<c10::StreamId>(((static_cast<uint64_t>(p) * kStreamsPerPool + i) << 1) | 1);
  return Stream(make(device, id));
}

Stream get_stream_from_pool(bool high_priority, c10::DeviceIndex device) {
  init_priorities();
  return get_stream_from_pool(high_priority ? -(g_num_prio - 1) : 0, device);
}

Stream get_stream_from_external(cudaStream_t ext, c10::DeviceIndex device) {
  device = resolve(device);
  if (ext == nullptr) return get_default_stream(device);
  auto v = reinterpret_cast<uintptr_t>(ext);
  TORCH_CHECK((v & 1) == 0, "external stream handle must be even-aligned");
  return Stream(make(device, static_cast<c10::StreamId>(v)));
}

Stream get_default_stream(c10::DeviceIndex device) { return Stream(make(resolve(device), 0)); }

Stream get_current_stream(c10::DeviceIndex device) {
  device = resolve(device);
  return Stream(make(device, tl_current[device]));
}

void set_current_stream(Stream s) { tl_current[s.device_index()] = s.id(); }

// ------------------------------------------------------------------ Event
// ---- event cache: creating and destroying a cudaEvent per collective / per freed block costs microseconds
// each; finished events go back to a per-(device, flags) free list instead (B200_EVENT_CACHE=0 or
// BCCL_ENABLE_EVENT_CACHE=0 switches it off).  Inter-process events are never cached: their handles were
// given to other processes.  Parity: reference torch_musa/csrc/distributed/ProcessGroupMCCL.cpp (MUSAEventCache).
namespace {
struct EventCache {
  std::mutex mu;
  std::map<std::pair<int, unsigned>, std::vector<cudaEvent_t>> free_list;
  std::atomic<int64_t> hits{0}, misses{0};
  bool enabled = [] {
    for (const char* n : {"B200_EVENT_CACHE", "BCCL_ENABLE_EVENT_CACHE"})
      if (const char* e = std::getenv(n)) return std::atoi(e) != 0;
    return true;
  }();
  static constexpr size_t kMaxPerKey = 1024;
};
EventCache& event_cache() {
  static EventCache* c = new EventCache();  // leaked: events may be destroyed during static destruction
  return *c;
}
}  // namespace

std::pair<int64_t, int64_t> event_cache_stats() {
  auto& c = event_cache();
  return {c.hits.load(), c.misses.load()};
}

Event::~Event() { destroy(); }

void Event::destroy() noexcept {
  if (created_) {
    auto& c = event_cache();
    if (c.enabled && !(flags_ & cudaEventInterprocess)) {
      std::lock_guard<std::mutex> g(c.mu);
      auto& v = c.free_list[{(int)device_, flags_}];
      if (v.size() < EventCache::kMaxPerKey) {
        v.push_back(ev_);
        created_ = false;
        return;
      }
    }
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != device_) cudaSetDevice(device_);
    B200_CUDA_WARN(cudaEventDestroy(ev_));
    if (cur != device_ && cur >= 0) cudaSetDevice(cur);
    created_ = false;
  }
}

void Event::move_from(Event&& o) noexcept {
  flags_ = o.flags_;
  created_ = o.created_;
  recorded_ = o.recorded_;
  device_ = o.device_;
  ev_ = o.ev_;
  o.created_ = false;
  o.ev_ = nullptr;
}

void Event::create(c10::DeviceIndex d) {
  auto& c = event_cache();
  if (c.enabled && !(flags_ & cudaEventInterprocess)) {
    std::lock_guard<std::mutex> g(c.mu);
    auto it = c.free_list.find({(int)d, flags_});
    if (it != c.free_list.end() && !it->second.empty()) {
      ev_ = it->second.back();
      it->second.pop_back();
      device_ = d;
      created_ = true;
      recorded_ = false;
      c.hits.fetch_add(1, std::memory_order_relaxed);
      return;
    }
  }
  c.misses.fetch_add(1, std::memory_order_relaxed);
  DeviceSwitch sw(d);
  B200_CUDA_CHECK(cudaEventCreateWithFlags(&ev_, flags_));
  device_ = d;
  created_ = true;
}

bool Event::query() const {
  if (!created_) return true;
  cudaError_t e = cudaEventQuery(ev_);
  if (e == cudaSuccess) return true;
  if (e != cudaErrorNotReady) B200_CUDA_CHECK(e);
  (void)cudaGetLastError();
  return false;
}

void Event::record() { record(get_current_stream()); }

void Event::record(const Stream& s) {
  if (!created_) create(s.device_index());
  TORCH_CHECK(device_ == s.device_index(), "Event device ", (int)device_, " does not match recording stream's device ",
              (int)s.device_index());
  DeviceSwitch sw(device_);
  B200_CUDA_CHECK(cudaEventRecord(ev_, s.stream()));
  recorded_ = true;
}

void Event::record_once(const Stream& s) {
  if (!recorded_) record(s);
}

void Event::block(const Stream& s) const {
  if (!created_) return;
  DeviceSwitch sw(s.device_index());
  B200_CUDA_CHECK(cudaStreamWaitEvent(s.stream(), ev_, 0));
}

void Event::synchronize() const {
  if (!created_) return;
  note_implicit_sync("Event::synchronize");
  B200_CUDA_CHECK(cudaEventSynchronize(ev_));
}

float Event::elapsed_ms(const Event& later) const {
  TORCH_CHECK(created_ && later.created_, "both events must be recorded before calculating elapsed time");
  float ms = 0.f;
  B200_CUDA_CHECK(cudaEventElapsedTime(&ms, ev_, later.ev_));
  return ms;
}

void Event::ipc_handle(cudaIpcEventHandle_t* out) {
  if (!created_) create(current_device());
  DeviceSwitch sw(device_);
  B200_CUDA_CHECK(cudaIpcGetEventHandle(out, ev_));
}

Event Event::from_ipc_handle(c10::DeviceIndex device, const cudaIpcEventHandle_t* h) {
  Event e(cudaEventDisableTiming | cudaEventInterprocess);
  DeviceSwitch sw(device);
  B200_CUDA_CHECK(cudaIpcOpenEventHandle(&e.ev_, *h));
  e.device_ = device;
  e.created_ = true;
  e.recorded_ = true;
  return e;
}

StreamGuard::StreamGuard(Stream s)
    : prev_device_(exchange_device(s.device_index())), prev_stream_(get_current_stream(s.device_index())) {
  set_current_stream(s);
}

StreamGuard::~StreamGuard() {
  set_current_stream(prev_stream_);
  cudaSetDevice(prev_device_);
}

}  // namespace b200
