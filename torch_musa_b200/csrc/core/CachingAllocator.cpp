#include "core/CachingAllocator.h"

#include <c10/util/Backtrace.h>
#include <c10/util/Exception.h>
#include <c10/util/irange.h>

#include <cuda.h>
#include <sys/mman.h>
#include <unistd.h>

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
size_t host_cap();
int host_alloc(void** p, size_t n, int, cudaStream_t) {
  *p = nullptr;
  // An artificial ceiling lets the tests exercise the OOM/retry path without a GPU.
  if (g_host_in_use + n > host_cap()) return (int)cudaErrorMemoryAllocation;
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

size_t host_cap() {
  static const size_t cap = [] {
    const char* e = std::getenv("B200_HOST_BACKEND_CAP_MB");
    return e ? (size_t)std::atoll(e) << 20 : (size_t)1 << 40;
  }();
  return cap;
}

// ---- host VMM: address space from mmap(PROT_NONE), "physical" chunks by mprotect.
size_t host_vmm_granularity(int) { return 2u << 20; }
int host_vmm_reserve(void** va, size_t n, int) {
  void* p = mmap(nullptr, n, PROT_NONE, MAP_PRIVATE | MAP_ANONYMOUS | MAP_NORESERVE, -1, 0);
  if (p == MAP_FAILED) return (int)cudaErrorMemoryAllocation;
  *va = p;
  return 0;
}
int host_vmm_release(void* va, size_t n, int) { return munmap(va, n) == 0 ? 0 : (int)cudaErrorInvalidValue; }
int host_vmm_map(void* va, size_t n, int, uint64_t* handle) {
  if (g_host_in_use + n > host_cap()) return (int)cudaErrorMemoryAllocation;
  if (mprotect(va, n, PROT_READ | PROT_WRITE) != 0) return (int)cudaErrorMemoryAllocation;
  g_host_in_use += n;
  *handle = (uint64_t)(uintptr_t)va | 1u;  // non-zero token
  return 0;
}
int host_vmm_unmap(void* va, size_t n, int, uint64_t) {
  madvise(va, n, MADV_DONTNEED);
  if (mprotect(va, n, PROT_NONE) != 0) return (int)cudaErrorInvalidValue;
  g_host_in_use -= n;
  return 0;
}
const VmmOps kHostVmm{host_vmm_granularity, host_vmm_reserve, host_vmm_release, host_vmm_map, host_vmm_unmap,
                      nullptr, nullptr};

// ---- CUDA VMM: the driver's cuMem* calls, looked up through the runtime so that
// nothing links against libcuda (the package must import on machines without a driver).
struct DriverVmm {
  decltype(&cuMemAddressReserve) address_reserve = nullptr;
  decltype(&cuMemAddressFree) address_free = nullptr;
  decltype(&cuMemCreate) create = nullptr;
  decltype(&cuMemRelease) release = nullptr;
  decltype(&cuMemMap) map = nullptr;
  decltype(&cuMemUnmap) unmap = nullptr;
  decltype(&cuMemSetAccess) set_access = nullptr;
  decltype(&cuMemGetAllocationGranularity) granularity = nullptr;
  decltype(&cuMemExportToShareableHandle) export_handle = nullptr;
  decltype(&cuMemImportFromShareableHandle) import_handle = nullptr;
  bool ok = false;
  bool fd_handles = true;  // cleared when the driver refuses shareable allocations
};
const DriverVmm& driver_vmm() {
  static DriverVmm d = [] {
    DriverVmm v;
    auto get = [](const char* name, void** fn) {
      cudaDriverEntryPointQueryResult q;
      cudaError_t e = cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q);
      if (e != cudaSuccess) (void)cudaGetLastError();
      return e == cudaSuccess && q == cudaDriverEntryPointSuccess && *fn != nullptr;
    };
    v.ok = get("cuMemAddressReserve", (void**)&v.address_reserve) && get("cuMemAddressFree", (void**)&v.address_free) &&
           get("cuMemCreate", (void**)&v.create) && get("cuMemRelease", (void**)&v.release) &&
           get("cuMemMap", (void**)&v.map) && get("cuMemUnmap", (void**)&v.unmap) &&
           get("cuMemSetAccess", (void**)&v.set_access) &&
           get("cuMemGetAllocationGranularity", (void**)&v.granularity) &&
           get("cuMemExportToShareableHandle", (void**)&v.export_handle) &&
           get("cuMemImportFromShareableHandle", (void**)&v.import_handle);
    return v;
  }();
  return d;
}
bool g_vmm_fd_handles = true;
CUmemAllocationProp vmm_prop(int device, bool fd) {
  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device;
  prop.requestedHandleTypes = fd ? CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR : CU_MEM_HANDLE_TYPE_NONE;
  return prop;
}
int vmm_err(CUresult r) {
  if (r == CUDA_SUCCESS) return 0;
  if (r == CUDA_ERROR_OUT_OF_MEMORY) return (int)cudaErrorMemoryAllocation;
  return (int)cudaErrorUnknown;
}
size_t cuda_vmm_granularity(int device) {
  const DriverVmm& d = driver_vmm();
  if (!d.ok) return 0;
  CUmemAllocationProp prop = vmm_prop(device, false);
  size_t g = 0;
  if (d.granularity(&g, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS) return 0;
  return g;
}
int cuda_vmm_reserve(void** va, size_t n, int) {
  CUdeviceptr p = 0;
  CUresult r = driver_vmm().address_reserve(&p, n, 0, 0, 0);
  *va = reinterpret_cast<void*>(p);
  return vmm_err(r);
}
int cuda_vmm_release(void* va, size_t n, int) { return vmm_err(driver_vmm().address_free((CUdeviceptr)va, n)); }
int cuda_vmm_access(void* va, size_t n, int device) {
  // Read/write for the owning GPU and for every GPU that has peer access to it switched on.
  std::vector<CUmemAccessDesc> descs;
  int ndev = device_count();
  for (int d = 0; d < ndev; ++d) {
    if (d != device && !peer_access_enabled((c10::DeviceIndex)d, (c10::DeviceIndex)device)) continue;
    CUmemAccessDesc a{};
    a.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    a.location.id = d;
    a.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    descs.push_back(a);
  }
  return vmm_err(driver_vmm().set_access((CUdeviceptr)va, n, descs.data(), descs.size()));
}
int cuda_vmm_map(void* va, size_t n, int device, uint64_t* handle) {
  const DriverVmm& d = driver_vmm();
  CUmemGenericAllocationHandle h = 0;
  CUmemAllocationProp prop = vmm_prop(device, g_vmm_fd_handles);
  CUresult r = d.create(&h, n, &prop, 0);
  if (g_vmm_fd_handles && (r == CUDA_ERROR_NOT_PERMITTED || r == CUDA_ERROR_NOT_SUPPORTED)) {
    g_vmm_fd_handles = false;  // containers without the capability: chunks stay process-private
    prop = vmm_prop(device, false);
    r = d.create(&h, n, &prop, 0);
  }
  if (r != CUDA_SUCCESS) return vmm_err(r);
  r = d.map((CUdeviceptr)va, n, 0, h, 0);
  if (r != CUDA_SUCCESS) {
    d.release(h);
    return vmm_err(r);
  }
  int e = cuda_vmm_access(va, n, device);
  if (e != 0) {
    d.unmap((CUdeviceptr)va, n);
    d.release(h);
    return e;
  }
  *handle = (uint64_t)h;
  return 0;
}
int cuda_vmm_unmap(void* va, size_t n, int, uint64_t handle) {
  const DriverVmm& d = driver_vmm();
  CUresult r = d.unmap((CUdeviceptr)va, n);
  if (r != CUDA_SUCCESS) return vmm_err(r);
  return vmm_err(d.release((CUmemGenericAllocationHandle)handle));
}
int cuda_vmm_export(uint64_t handle, int* fd) {
  if (!g_vmm_fd_handles) return (int)cudaErrorNotSupported;
  return vmm_err(driver_vmm().export_handle(fd, (CUmemGenericAllocationHandle)handle,
                                            CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
}
int cuda_vmm_import(int fd, void* va, size_t n, int device, uint64_t* handle) {
  const DriverVmm& d = driver_vmm();
  CUmemGenericAllocationHandle h = 0;
  CUresult r = d.import_handle(&h, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
  if (r != CUDA_SUCCESS) return vmm_err(r);
  r = d.map((CUdeviceptr)va, n, 0, h, 0);
  if (r != CUDA_SUCCESS) {
    d.release(h);
    return vmm_err(r);
  }
  int e = cuda_vmm_access(va, n, device);
  if (e != 0) {
    d.unmap((CUdeviceptr)va, n);
    d.release(h);
    return e;
  }
  *handle = (uint64_t)h;
  return 0;
}
const VmmOps kCudaVmm{cuda_vmm_granularity, cuda_vmm_reserve, cuda_vmm_release, cuda_vmm_map, cuda_vmm_unmap,
                      cuda_vmm_export, cuda_vmm_import};

const RawBackend kNative{"native", native_alloc, native_free, cuda_mem_info, true, &kCudaVmm};
const RawBackend kUnified{"unified", unified_alloc, native_free, cuda_mem_info, true, nullptr};
const RawBackend kAsync{"cudaMallocAsync", async_alloc, async_free, cuda_mem_info, true, nullptr};
const RawBackend kHost{"host", host_alloc, host_free, host_mem_info, false, &kHostVmm};
RawBackend g_plug{"pluggable", nullptr, nullptr, cuda_mem_info, true, nullptr};

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
    } else if (k == "canary") {
      c.canary = parse_bool(k, v);
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
struct XSegment;
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
  bool has_canary = false;   // guard bytes sit behind `requested`
  XSegment* xseg = nullptr;  // expandable segment this block lies in
  bool mapped = true;        // false: address space only (never in Pool::blocks)
  bool is_split() const { return prev || next; }
};

// Address-ordered set of the unmapped ranges of a pool's expandable segments.
struct UnmappedLess {
  bool operator()(const Block* a, const Block* b) const {
    if (a->stream != b->stream) return (uintptr_t)a->stream < (uintptr_t)b->stream;
    return (uintptr_t)a->ptr < (uintptr_t)b->ptr;
  }
};

// One reserved address range that grows and shrinks in `unit`-sized physical chunks.
struct XSegment {
  char* base = nullptr;
  size_t reserved = 0, unit = 0, mapped_bytes = 0;
  cudaStream_t stream = nullptr;
  Pool* pool = nullptr;
  std::vector<uint64_t> handles;  // one per unit; 0 = not mapped
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
  std::set<Block*, UnmappedLess> unmapped;
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

  // ---- guard bytes (debug option `canary:True`): kCanaryBytes of a fixed pattern directly behind the requested
  // bytes of every allocation, checked when the allocation is freed.  An out-of-bounds write of a kernel then
  // shows up at the free of the block it overran, with the block's size, instead of as silent corruption of a
  // neighbour.  Costs a memset per allocation and a synchronous 64-byte read-back per free.
  static constexpr size_t kCanaryBytes = 64;
  static constexpr unsigned char kCanaryByte = 0xA5;

  void write_canary(Block* b) {
    char* at = static_cast<char*>(b->ptr) + b->requested;
    if (be_->device_events) {
      DeviceSwitch sw(device_);
      B200_CUDA_WARN(cudaMemsetAsync(at, kCanaryByte, kCanaryBytes, b->stream));
    } else {
      std::memset(at, kCanaryByte, kCanaryBytes);
    }
  }
  void check_canary(Block* b) {
    unsigned char host[kCanaryBytes];
    const char* at = static_cast<const char*>(b->ptr) + b->requested;
    if (be_->device_events) {
      DeviceSwitch sw(device_);
      if (cudaMemcpy(host, at, kCanaryBytes, cudaMemcpyDeviceToHost) != cudaSuccess) {
        (void)cudaGetLastError();
        return;
      }
    } else {
      std::memcpy(host, at, kCanaryBytes);
    }
    for (size_t i = 0; i < kCanaryBytes; ++i) {
      if (host[i] != kCanaryByte) {
        ++canary_violations_;
        std::ostringstream os;
        os << "blackwell allocator: the " << b->requested << "-byte allocation at " << b->ptr << " (device " << device_
           << ") was written " << (i + 1) << " or more bytes past its end";
        canary_report_ = os.str();
        TORCH_WARN(canary_report_);
        return;
      }
    }
  }

  Block* malloc(size_t orig, cudaStream_t stream) {
    std::unique_lock<std::mutex> lk(mu_);
    process_events();
    const bool canary = config().canary;
    size_t size = round_size(orig + (canary ? kCanaryBytes : 0));
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
      rem->xseg = b->xseg;
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
    mark_allocated(b, orig);
    b->has_canary = canary;
    if (canary) write_canary(b);
    return b;
  }

  void mark_allocated(Block* b, size_t requested) {
    Pool& pool = *b->pool;
    b->allocated = true;
    b->requested = requested;
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
    trace(TraceEntry::ALLOC, b->ptr, b->size, b->stream);
  }

  void free(Block* b) {
    std::lock_guard<std::mutex> lk(mu_);
    free_locked(b, /*ignore_stream_uses=*/false);
  }

  void free_locked(Block* b, bool ignore_stream_uses) {
    if (ignore_stream_uses) b->stream_uses.clear();
    if (b->has_canary) {
      check_canary(b);
      b->has_canary = false;
    }
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
      // An expandable segment reports each run of mapped blocks as a segment of its own.
      Block* b = h;
      while (b) {
        while (b && !b->mapped) b = b->next;
        if (!b) break;
        SegmentInfo s;
        s.device = device_;
        s.address = (uintptr_t)b->ptr;
        s.stream = b->stream;
        s.is_large = !b->pool->is_small;
        s.is_expandable = b->xseg != nullptr;
        s.pool_id_first = id.first;
        s.pool_id_second = id.second;
        for (; b && b->mapped; b = b->next) {
          s.total_size += b->size;
          BlockInfo bi;
          bi.address = (uintptr_t)b->ptr;
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
    }
    std::sort(out.begin(), out.end(), [](const SegmentInfo& a, const SegmentInfo& b) { return a.address < b.address; });
    trace(TraceEntry::SNAPSHOT, nullptr, 0, nullptr);
    return out;
  }

  // Puts the private pool `state.pool` back into the block layout of the checkpoint: everything live in it is
  // freed, then each checkpointed segment is carved into the recorded blocks and the ones that were allocated
  // become live again at their old addresses.
  RestoreResult restore(const PoolCheckpoint& state) {
    std::lock_guard<std::mutex> lk(mu_);
    auto pit = private_.find(state.pool);
    TORCH_CHECK(pit != private_.end(), "restore_pool: the pool of this checkpoint no longer exists");
    PrivatePool* pp = pit->second.get();
    TORCH_CHECK(capturing_depth_ == 0, "restore_pool cannot run while a capture is under way");
    sync_and_drain();
    std::vector<Block*> mine;
    for (auto& kv : live_) if (kv.second->pool->owner == pp) mine.push_back(kv.second);
    std::set<void*> was_live;
    ++pp->use_count;  // a pool nobody captures into any more must not hand its segments back half-way through
    for (Block* b : mine) {
      was_live.insert(b->ptr);
      free_locked(b, /*ignore_stream_uses=*/true);
    }
    --pp->use_count;
    RestoreResult res;
    for (const SegmentInfo& seg : state.segments) {
      Pool& pool = seg.is_large ? pp->large : pp->small;
      char* lo = reinterpret_cast<char*>(seg.address);
      Block* f = nullptr;
      for (Block* b : pool.blocks) {
        if (static_cast<char*>(b->ptr) <= lo && static_cast<char*>(b->ptr) + b->size >= lo + seg.total_size) {
          f = b;
          break;
        }
      }
      TORCH_CHECK(f, "restore_pool: the segment at ", (void*)lo, " (", seg.total_size,
                  " bytes) is no longer a free range of the pool");
      pool.blocks.erase(f);
      if (f->is_split()) bump([&](int t) { stats_.inactive_split[t].dec(1); stats_.inactive_split_bytes[t].dec(f->size); }, pool);
      auto put_free = [&](Block* b) {
        pool.blocks.insert(b);
        if (b->is_split()) bump([&](int t) { stats_.inactive_split[t].inc(1); stats_.inactive_split_bytes[t].inc(b->size); }, pool);
      };
      // cuts the first `n` bytes off `b`; returns the rest (linked, in no set) or null when nothing is left
      auto cut = [&](Block* b, size_t n) -> Block* {
        if (b->size == n) return nullptr;
        Block* rem = new Block();
        rem->device = device_;
        rem->stream = b->stream;
        rem->pool = &pool;
        rem->xseg = b->xseg;
        rem->ptr = static_cast<char*>(b->ptr) + n;
        rem->size = b->size - n;
        rem->prev = b;
        rem->next = b->next;
        if (rem->next) rem->next->prev = rem;
        b->next = rem;
        b->size = n;
        return rem;
      };
      if (static_cast<char*>(f->ptr) < lo) {  // an expandable range that has grown downwards since
        Block* rest = cut(f, (size_t)(lo - static_cast<char*>(f->ptr)));
        put_free(f);
        f = rest;
      }
      for (const BlockInfo& bi : seg.blocks) {
        TORCH_INTERNAL_ASSERT(f && (uintptr_t)f->ptr == bi.address && f->size >= bi.size);
        Block* rest = cut(f, bi.size);
        if (bi.allocated) {
          mark_allocated(f, bi.requested);
          res.allocated.push_back(f->ptr);
        } else {
          put_free(f);
        }
        f = rest;
      }
      if (f) put_free(f);
    }
    std::set<void*> now(res.allocated.begin(), res.allocated.end());
    for (void* p : was_live) if (!now.count(p)) res.freed.push_back(p);
    return res;
  }

  bool share(void* p, CachingAllocator::ShareInfo* out) {
    std::lock_guard<std::mutex> lk(mu_);
    auto it = live_.upper_bound(p);
    if (it == live_.begin()) return false;
    --it;
    Block* b = it->second;
    if (static_cast<char*>(p) >= static_cast<char*>(b->ptr) + b->size) return false;
    if (!b->xseg || !be_->vmm->export_fd) return false;
    XSegment* xs = b->xseg;
    size_t off = (size_t)(static_cast<char*>(p) - xs->base);
    size_t len = b->size - (size_t)(static_cast<char*>(p) - static_cast<char*>(b->ptr));
    size_t first = off / xs->unit, last = (off + len - 1) / xs->unit;
    out->fds.clear();
    for (size_t i = first; i <= last; ++i) {
      int fd = -1;
      if (be_->vmm->export_fd(xs->handles[i], &fd) != 0) {
        if (be_->device_events) (void)cudaGetLastError();
        for (int f : out->fds) ::close(f);
        out->fds.clear();
        return false;
      }
      out->fds.push_back(fd);
    }
    out->chunk_bytes = xs->unit;
    out->offset = off - first * xs->unit;
    out->size = len;
    return true;
  }

  void refresh_peer_access() {
    std::lock_guard<std::mutex> lk(mu_);
    DeviceSwitch sw(be_->device_events ? device_ : -1);
    refresh_peer_access_locked();
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

  void set_history(bool on, size_t max_entries, bool stacks = false) {
    std::lock_guard<std::mutex> lk(mu_);
    history_stacks_ = on && stacks;
    history_ = on;
    history_max_ = max_entries ? max_entries : 1;
    if (!on) trace_.clear();
  }
  std::vector<TraceEntry> get_trace() {
    std::lock_guard<std::mutex> lk(mu_);
    return std::vector<TraceEntry>(trace_.begin(), trace_.end());
  }

  std::vector<OomObserver>* observers = nullptr;
  int64_t canary_violations() {
    std::lock_guard<std::mutex> lk(mu_);
    return canary_violations_;
  }
  std::string canary_report() {
    std::lock_guard<std::mutex> lk(mu_);
    return canary_report_;
  }

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
    trace_.push_back(TraceEntry{a, device_, (uintptr_t)p, n, s, now_ns(), {}});
    // symbolised C++ frames of the caller (allocation sites); only while asked for: it costs tens of microseconds
    if (history_stacks_ && (a == TraceEntry::ALLOC || a == TraceEntry::SEGMENT_ALLOC || a == TraceEntry::OOM))
      trace_.back().stack = c10::get_backtrace(/*frames_to_skip=*/3, /*maximum_number_of_frames=*/20);
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

  // ------------------------------------------------- expandable segments
  bool use_expandable() const { return config().expandable_segments && be_->vmm != nullptr; }

  bool is_free_mapped(const Block* b) const {
    return b && b->mapped && !b->allocated && b->event_count == 0 && b->stream_uses.empty() &&
           b->pool->blocks.count(const_cast<Block*>(b));
  }

  XSegment* new_xsegment(Pool& pool, cudaStream_t stream) {
    size_t gran = be_->vmm->granularity(device_);
    if (gran == 0) return nullptr;
    size_t unit = pool.is_small ? kSmallBuffer : std::max(config().large_segment_bytes, (size_t)(20u << 20));
    unit = (unit + gran - 1) / gran * gran;
    size_t fr = 0, tot = 0;
    if (be_->mem_info(device_, &fr, &tot) != 0 || tot == 0) return nullptr;
    // Room for the whole device plus slack: a segment never has to move.
    size_t reserve = (tot + tot / 8 + unit - 1) / unit * unit;
    void* va = nullptr;
    if (be_->vmm->reserve(&va, reserve, device_) != 0) {
      if (be_->device_events) (void)cudaGetLastError();
      return nullptr;
    }
    auto xs = std::make_unique<XSegment>();
    xs->base = static_cast<char*>(va);
    xs->reserved = reserve;
    xs->unit = unit;
    xs->stream = stream;
    xs->pool = &pool;
    xs->handles.assign(reserve / unit, 0);
    Block* u = new Block();
    u->device = device_;
    u->stream = stream;
    u->pool = &pool;
    u->ptr = va;
    u->size = reserve;
    u->xseg = xs.get();
    u->mapped = false;
    pool.unmapped.insert(u);
    xsegs_.push_back(std::move(xs));
    return xsegs_.back().get();
  }

  // Maps the first `bytes` (rounded up to whole units) of the unmapped block `u`; returns the new
  // free mapped block (merged with a free mapped predecessor), not inserted in the pool.
  Block* map_front(Block* u, size_t bytes) {
    XSegment* xs = u->xseg;
    Pool& pool = *u->pool;
    bytes = (bytes + xs->unit - 1) / xs->unit * xs->unit;
    if (bytes > u->size) return nullptr;
    if (limited_ && (size_t)stats_.reserved_bytes[kAll].current + bytes > allowed_) return nullptr;
    size_t first = (size_t)(static_cast<char*>(u->ptr) - xs->base) / xs->unit, n = bytes / xs->unit, done = 0;
    int e = 0;
    for (; done < n; ++done) {
      e = be_->vmm->map(xs->base + (first + done) * xs->unit, xs->unit, device_, &xs->handles[first + done]);
      if (e != 0) break;
    }
    if (e != 0) {
      if (be_->device_events) (void)cudaGetLastError();
      for (size_t i = 0; i < done; ++i) {
        be_->vmm->unmap(xs->base + (first + i) * xs->unit, xs->unit, device_, xs->handles[first + i]);
        xs->handles[first + i] = 0;
      }
      if (e != (int)cudaErrorMemoryAllocation) check_cuda((cudaError_t)e, "expandable segment map", __FILE__, __LINE__);
      return nullptr;
    }
    ++stats_.num_device_alloc;
    if (xs->mapped_bytes == 0) bump([&](int t) { stats_.segment[t].inc(1); }, pool);
    xs->mapped_bytes += bytes;
    bump([&](int t) { stats_.reserved_bytes[t].inc(bytes); }, pool);
    trace(TraceEntry::SEGMENT_ALLOC, u->ptr, bytes, u->stream);
    // carve [u->ptr, u->ptr + bytes) off the front of u
    Block* m = new Block();
    m->device = device_;
    m->stream = u->stream;
    m->pool = &pool;
    m->xseg = xs;
    m->ptr = u->ptr;
    m->size = bytes;
    m->prev = u->prev;
    if (m->prev) m->prev->next = m;
    pool.unmapped.erase(u);
    if (u->size == bytes) {
      m->next = u->next;
      if (m->next) m->next->prev = m;
      delete u;
    } else {
      u->ptr = static_cast<char*>(u->ptr) + bytes;
      u->size -= bytes;
      u->prev = m;
      m->next = u;
      pool.unmapped.insert(u);
    }
    // join free mapped neighbours (the successor can be one when a hole was re-mapped)
    for (Block* nb : {m->prev, m->next}) {
      if (!is_free_mapped(nb)) continue;
      pool.blocks.erase(nb);
      bump([&](int t) { stats_.inactive_split[t].dec(1); stats_.inactive_split_bytes[t].dec(nb->size); }, pool);
      if (nb == m->prev) {
        m->ptr = nb->ptr;
        m->prev = nb->prev;
        if (m->prev) m->prev->next = m;
      } else {
        m->next = nb->next;
        if (m->next) m->next->prev = m;
      }
      m->size += nb->size;
      delete nb;
    }
    return m;
  }

  Block* alloc_expandable(Pool& pool, size_t size, cudaStream_t stream) {
    Block key;
    key.stream = stream;
    key.ptr = nullptr;
    for (auto it = pool.unmapped.lower_bound(&key); it != pool.unmapped.end() && (*it)->stream == stream; ++it) {
      Block* u = *it;
      size_t have = is_free_mapped(u->prev) ? u->prev->size : 0;
      size_t need = size > have ? size - have : u->xseg->unit;
      size_t rounded = (need + u->xseg->unit - 1) / u->xseg->unit * u->xseg->unit;
      if (rounded > u->size) continue;
      // A hole between mapped ranges has to be filled whole or the result would not be contiguous enough.
      return map_front(u, need);
    }
    XSegment* xs = new_xsegment(pool, stream);
    if (!xs) return nullptr;
    Block k2;
    k2.stream = stream;
    k2.ptr = xs->base;
    auto it = pool.unmapped.find(&k2);
    if (it == pool.unmapped.end()) return nullptr;
    Block* m = map_front(*it, size);
    if (!m) drop_if_empty(xs);
    return m;
  }

  // Releases the address range of a segment with nothing mapped.
  void drop_if_empty(XSegment* xs) {
    if (xs->mapped_bytes != 0) return;
    Pool& pool = *xs->pool;
    Block k;
    k.stream = xs->stream;
    k.ptr = xs->base;
    auto it = pool.unmapped.find(&k);
    if (it == pool.unmapped.end() || (*it)->size != xs->reserved) return;
    Block* u = *it;
    pool.unmapped.erase(it);
    delete u;
    be_->vmm->release(xs->base, xs->reserved, device_);
    for (auto i = xsegs_.begin(); i != xsegs_.end(); ++i) {
      if (i->get() == xs) {
        xsegs_.erase(i);
        break;
      }
    }
  }

  // Unmaps the whole units inside the free mapped block `b` (which sits in its pool).  Returns the bytes given back.
  size_t unmap_block(Block* b) {
    XSegment* xs = b->xseg;
    Pool& pool = *b->pool;
    size_t off = (size_t)(static_cast<char*>(b->ptr) - xs->base);
    size_t lo = (off + xs->unit - 1) / xs->unit * xs->unit;
    size_t hi = (off + b->size) / xs->unit * xs->unit;
    if (hi <= lo) return 0;
    if (be_->device_events) {
      // Work queued on the block's stream may still touch it: unmapping, unlike cudaFree, does not wait.
      DeviceSwitch sw(device_);
      B200_CUDA_CHECK(cudaStreamSynchronize(b->stream));
    }
    pool.blocks.erase(b);
    if (b->is_split()) bump([&](int t) { stats_.inactive_split[t].dec(1); stats_.inactive_split_bytes[t].dec(b->size); }, pool);
    for (size_t i = lo / xs->unit; i < hi / xs->unit; ++i) {
      B200_KERNEL_CALL(be_->vmm->unmap(xs->base + i * xs->unit, xs->unit, device_, xs->handles[i]));
      xs->handles[i] = 0;
    }
    size_t bytes = hi - lo;
    ++stats_.num_device_free;
    xs->mapped_bytes -= bytes;
    bump([&](int t) { stats_.reserved_bytes[t].dec(bytes); }, pool);
    if (xs->mapped_bytes == 0) bump([&](int t) { stats_.segment[t].dec(1); }, pool);
    trace(TraceEntry::SEGMENT_FREE, xs->base + lo, bytes, b->stream);
    // b becomes [head mapped][middle unmapped][tail mapped]
    size_t head = lo - off, tail = off + b->size - hi;
    Block* mid = b;
    if (head) {
      Block* hb = new Block();
      hb->device = device_;
      hb->stream = b->stream;
      hb->pool = &pool;
      hb->xseg = xs;
      hb->ptr = b->ptr;
      hb->size = head;
      hb->prev = b->prev;
      if (hb->prev) hb->prev->next = hb;
      hb->next = mid;
      mid->prev = hb;
      pool.blocks.insert(hb);
      bump([&](int t) { stats_.inactive_split[t].inc(1); stats_.inactive_split_bytes[t].inc(head); }, pool);
    }
    if (tail) {
      Block* tb = new Block();
      tb->device = device_;
      tb->stream = b->stream;
      tb->pool = &pool;
      tb->xseg = xs;
      tb->ptr = xs->base + hi;
      tb->size = tail;
      tb->next = b->next;
      if (tb->next) tb->next->prev = tb;
      tb->prev = mid;
      mid->next = tb;
      pool.blocks.insert(tb);
      bump([&](int t) { stats_.inactive_split[t].inc(1); stats_.inactive_split_bytes[t].inc(tail); }, pool);
    }
    mid->ptr = xs->base + lo;
    mid->size = bytes;
    mid->mapped = false;
    mid->gc_count = 0;
    // join neighbouring unmapped ranges
    for (Block* nb : {mid->prev, mid->next}) {
      if (!nb || nb->mapped) continue;
      pool.unmapped.erase(nb);
      if (nb == mid->prev) {
        mid->ptr = nb->ptr;
        mid->prev = nb->prev;
        if (mid->prev) mid->prev->next = mid;
      } else {
        mid->next = nb->next;
        if (mid->next) mid->next->prev = mid;
      }
      mid->size += nb->size;
      delete nb;
    }
    pool.unmapped.insert(mid);
    drop_if_empty(xs);
    return bytes;
  }

  void refresh_peer_access_locked() {
    if (!be_->vmm || !be_->device_events) return;
    for (auto& xs : xsegs_)
      for (size_t i = 0; i < xs->handles.size(); ++i)
        if (xs->handles[i]) B200_CUDA_WARN((cudaError_t)cuda_vmm_access(xs->base + i * xs->unit, xs->unit, device_));
  }

  Block* alloc_segment(Pool& pool, size_t size, cudaStream_t stream) {
    if (use_expandable()) {
      DeviceSwitch sw(be_->device_events ? device_ : -1);
      return alloc_expandable(pool, size, stream);
    }
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
      if (!b->is_split() && !b->xseg && b->size >= size) {
        sync_and_drain();
        release_block(b);
        return true;
      }
    }
    return false;
  }

  void release_pool_blocks(Pool& pool) {
    std::vector<Block*> whole, growable;
    for (Block* b : pool.blocks) {
      if (b->xseg) growable.push_back(b);
      else if (!b->is_split()) whole.push_back(b);
    }
    for (Block* b : whole) release_block(b);
    if (capturing_depth_ == 0) for (Block* b : growable) unmap_block(b);
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
    for (Block* b : large_.blocks) if (!b->is_split() && !b->xseg) { ++b->gc_count; cands.push_back(b); }
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
  std::vector<std::unique_ptr<XSegment>> xsegs_;
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
  int64_t canary_violations_ = 0;
  std::string canary_report_;
  bool history_ = false, history_stacks_ = false;
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
// A DataPtr's context is its data pointer; this table finds the allocator that owns it.
std::mutex g_ctx_mu;
std::unordered_map<void*, CachingAllocator*> g_ptr_owner;
bool g_pool_restored = false;  // a restore may leave DataPtrs behind whose memory it already took back

void deleter(void* ctx) {
  CachingAllocator* owner;
  {
    std::lock_guard<std::mutex> g(g_ctx_mu);
    auto it = g_ptr_owner.find(ctx);
    if (it == g_ptr_owner.end()) {
      TORCH_INTERNAL_ASSERT(g_pool_restored, "blackwell allocator: freeing an unknown pointer");
      return;
    }
    owner = it->second;
    g_ptr_owner.erase(it);
  }
  owner->raw_delete(ctx);
}
void noop(void*) {}

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
    g_ptr_owner[b->ptr] = this;
  }
  return c10::DataPtr(b->ptr, b->ptr, &deleter, make_device(device));
}

c10::DeleterFnPtr CachingAllocator::noop_deleter() { return &noop; }

c10::DataPtr CachingAllocator::adopt(void* p, int device) {
  TORCH_CHECK(device < (int)devs_.size() && devs_[device]->find_live(p), "blackwell allocator: ", p,
              " is not a live allocation on device ", device);
  {
    std::lock_guard<std::mutex> g(g_ctx_mu);
    TORCH_CHECK(!g_ptr_owner.count(p), "blackwell allocator: ", p, " already has an owner");
    g_ptr_owner[p] = this;
  }
  return c10::DataPtr(p, p, &deleter, make_device(device));
}

PoolCheckpoint CachingAllocator::checkpoint_pool(int device, MempoolId pool) {
  TORCH_CHECK(pool.first || pool.second, "checkpoint_pool needs a private pool id");
  PoolCheckpoint c;
  c.device = device;
  c.pool = pool;
  if (device < (int)devs_.size()) c.segments = devs_[device]->snapshot(pool);
  return c;
}

RestoreResult CachingAllocator::restore_pool(int device, const PoolCheckpoint& state) {
  TORCH_CHECK(device < (int)devs_.size() && state.device == device, "restore_pool: checkpoint of another device");
  RestoreResult r = devs_[device]->restore(state);
  std::lock_guard<std::mutex> g(g_ctx_mu);
  g_pool_restored = true;
  for (void* p : r.freed) g_ptr_owner.erase(p);
  return r;
}

bool CachingAllocator::share_expandable(void* p, ShareInfo* out) {
  for (auto& d : devs_)
    if (d->share(p, out)) return true;
  return false;
}

void* CachingAllocator::map_imported(const std::vector<int>& fds, size_t chunk, int device,
                                     std::vector<uint64_t>* handles) {
  const VmmOps* v = backend_->vmm;
  TORCH_CHECK(v && v->import_fd, "this allocator backend cannot import shared memory chunks");
  DeviceSwitch sw(backend_->device_events ? device : -1);
  void* va = nullptr;
  B200_KERNEL_CALL(v->reserve(&va, chunk * fds.size(), device));
  handles->assign(fds.size(), 0);
  for (size_t i = 0; i < fds.size(); ++i) {
    int e = v->import_fd(fds[i], static_cast<char*>(va) + i * chunk, chunk, device, &(*handles)[i]);
    if (e != 0) {
      for (size_t j = 0; j < i; ++j) v->unmap(static_cast<char*>(va) + j * chunk, chunk, device, (*handles)[j]);
      v->release(va, chunk * fds.size(), device);
      check_cuda((cudaError_t)e, "import of a shared memory chunk", __FILE__, __LINE__);
    }
  }
  return va;
}

void CachingAllocator::unmap_imported(void* va, size_t chunk, int device, const std::vector<uint64_t>& handles) {
  const VmmOps* v = backend_->vmm;
  DeviceSwitch sw(backend_->device_events ? device : -1);
  for (size_t i = 0; i < handles.size(); ++i)
    B200_CUDA_WARN((cudaError_t)v->unmap(static_cast<char*>(va) + i * chunk, chunk, device, handles[i]));
  B200_CUDA_WARN((cudaError_t)v->release(va, chunk * handles.size(), device));
}

void CachingAllocator::refresh_peer_access(int device) {
  if (device < (int)devs_.size()) devs_[device]->refresh_peer_access();
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
  for (auto& d : devs_) {
    if (Block* b = d->find_live(p.get())) {
      d->record_stream(b, stream);
      return;
    }
  }
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
      while (h->prev && h->prev->mapped) h = h->prev;
      size_t tot = 0;
      for (Block* x = h; x && x->mapped; x = x->next) tot += x->size;
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

int64_t CachingAllocator::canary_violations() const {
  int64_t n = 0;
  for (auto& d : devs_) n += d->canary_violations();
  return n;
}
std::string CachingAllocator::last_canary_report() const {
  for (auto& d : devs_) {
    std::string r = d->canary_report();
    if (!r.empty()) return r;
  }
  return {};
}

void CachingAllocator::attach_oom_observer(OomObserver o) { g_observers.push_back(std::move(o)); }
void CachingAllocator::record_history(bool enabled, size_t max_entries, bool stacks) {
  for (auto& d : devs_) d->set_history(enabled, max_entries, stacks);
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
    if (be->vmm && be->device_events)
      set_peer_access_hook([](int, int owner) { if (g_current) g_current->refresh_peer_access(owner); });
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
