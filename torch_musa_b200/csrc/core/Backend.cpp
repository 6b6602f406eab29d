// Registration of the blackwell backend with the framework: the device-guard
// implementation (device / stream / event switching used by DeviceGuard,
// torch.Stream and torch.Event), the PrivateUse1 hooks (lazy init, pinned
// allocator, generators, pointer queries, storage resize) and the device
// allocator.  Everything here runs at library load time and touches no GPU.
// Parity: reference torch_musa/csrc/core/GuardImpl.h:19-250, GuardImpl.cpp:5,
// MUSAHooks.cpp:17-99, MUSACachingAllocator.cpp:3478.
#include "core/Backend.h"

#include "core/CachingAllocator.h"
#include "core/Generator.h"
#include "core/HostAllocator.h"
#include "core/Stream.h"

#include <ATen/detail/PrivateUse1HooksInterface.h>
#include <c10/core/impl/DeviceGuardImplInterface.h>
#include <c10/core/impl/GPUTrace.h>
#include <c10/util/CallOnce.h>
#include <c10/util/Logging.h>

namespace b200 {

namespace {

struct GuardImpl final : public c10::impl::DeviceGuardImplInterface {
  c10::DeviceType type() const override { return kDeviceType; }

  c10::Device exchangeDevice(c10::Device d) const override {
    TORCH_INTERNAL_ASSERT(d.type() == kDeviceType);
    return make_device(exchange_device(d.index()));
  }
  c10::Device getDevice() const override {
    // Guards are constructed in generic code paths even on GPU-less hosts.
    if (device_count() == 0) return make_device(0);
    return make_device(current_device());
  }
  void setDevice(c10::Device d) const override {
    TORCH_INTERNAL_ASSERT(d.type() == kDeviceType);
    if (device_count() == 0) return;
    set_device(d.index());
  }
  void uncheckedSetDevice(c10::Device d) const noexcept override {
    if (device_count() == 0) return;
    B200_CUDA_WARN(cudaSetDevice(d.index()));
  }
  c10::Stream getStream(c10::Device d) const override { return get_current_stream(d.index()).unwrap(); }
  c10::Stream getDefaultStream(c10::Device d) const override { return get_default_stream(d.index()).unwrap(); }
  c10::Stream getStreamFromGlobalPool(c10::Device d, bool high) const override {
    return get_stream_from_pool(high, d.index()).unwrap();
  }
  c10::Stream getNewStream(c10::Device d, int priority) const override {
    return get_stream_from_pool(priority, d.index()).unwrap();
  }
  c10::Stream exchangeStream(c10::Stream s) const override {
    Stream ns(s);
    auto old = get_current_stream(s.device_index());
    set_current_stream(ns);
    return old.unwrap();
  }
  void* getStreamNativeHandle(const c10::Stream s) const override { return stream_from_c10(s); }
  c10::DeviceIndex deviceCount() const noexcept override { return device_count(); }

  // ---- events (the generic torch.Event goes through these)
  void destroyEvent(void* event, const c10::DeviceIndex device_index) const noexcept override {
    if (!event) return;
    int cur = -1;
    cudaGetDevice(&cur);
    if (cur != device_index) cudaSetDevice(device_index);
    if (auto* t = c10::impl::GPUTrace::get_trace())
      (*t)->trace_gpu_event_deletion(kDeviceType, reinterpret_cast<uintptr_t>(event));
    B200_CUDA_WARN(cudaEventDestroy(static_cast<cudaEvent_t>(event)));
    if (cur != device_index && cur >= 0) cudaSetDevice(cur);
  }
  void record(void** event, const c10::Stream& stream, const c10::DeviceIndex device_index,
              const c10::EventFlag flag) const override {
    TORCH_CHECK(device_index == -1 || device_index == stream.device_index(), "Event device index ", (int)device_index,
                " does not match recording stream's device index ", (int)stream.device_index(), ".");
    DeviceSwitch sw(stream.device_index());
    auto ev = static_cast<cudaEvent_t>(*event);
    if (!ev) {
      unsigned f = cudaEventDisableTiming;
      if (flag == c10::EventFlag::BACKEND_DEFAULT) f = cudaEventDefault;
      B200_CUDA_CHECK(cudaEventCreateWithFlags(&ev, f));
      if (auto* t = c10::impl::GPUTrace::get_trace())
        (*t)->trace_gpu_event_creation(kDeviceType, reinterpret_cast<uintptr_t>(ev));
    }
    cudaStream_t cs = stream_from_c10(stream);
    B200_CUDA_CHECK(cudaEventRecord(ev, cs));
    *event = ev;
    if (auto* t = c10::impl::GPUTrace::get_trace())
      (*t)->trace_gpu_event_record(kDeviceType, reinterpret_cast<uintptr_t>(ev), reinterpret_cast<uintptr_t>(cs));
  }
  void block(void* event, const c10::Stream& stream) const override {
    if (!event) return;
    DeviceSwitch sw(stream.device_index());
    cudaStream_t cs = stream_from_c10(stream);
    B200_CUDA_CHECK(cudaStreamWaitEvent(cs, static_cast<cudaEvent_t>(event), 0));
    if (auto* t = c10::impl::GPUTrace::get_trace())
      (*t)->trace_gpu_event_wait(kDeviceType, reinterpret_cast<uintptr_t>(event), reinterpret_cast<uintptr_t>(cs));
  }
  bool queryEvent(void* event) const override {
    if (!event) return true;
    cudaError_t e = cudaEventQuery(static_cast<cudaEvent_t>(event));
    if (e == cudaErrorNotReady) {
      (void)cudaGetLastError();
      return false;
    }
    B200_CUDA_CHECK(e);
    return true;
  }
  bool queryStream(const c10::Stream& stream) const override { return Stream(stream).query(); }
  void synchronizeStream(const c10::Stream& stream) const override { Stream(stream).synchronize(); }
  void synchronizeEvent(void* event) const override {
    if (!event) return;
    note_implicit_sync("synchronizeEvent");
    B200_CUDA_CHECK(cudaEventSynchronize(static_cast<cudaEvent_t>(event)));
  }
  void synchronizeDevice(const c10::DeviceIndex device_index) const override {
    DeviceSwitch sw(device_index);
    device_synchronize();
  }
  void recordDataPtrOnStream(const c10::DataPtr& data_ptr, const c10::Stream& stream) const override {
    alloc::get()->record_stream(data_ptr, stream.device_index(), stream_from_c10(stream));
  }
  double elapsedTime(void* event1, void* event2, const c10::DeviceIndex device_index) const override {
    TORCH_CHECK(event1 && event2, "Both events must be recorded before calculating elapsed time.");
    DeviceSwitch sw(device_index);
    float ms = 0.f;
    B200_CUDA_CHECK(cudaEventElapsedTime(&ms, static_cast<cudaEvent_t>(event1), static_cast<cudaEvent_t>(event2)));
    return ms;
  }
};

C10_REGISTER_GUARD_IMPL(PrivateUse1, GuardImpl);

// The allocator object looked up by c10::GetAllocator(PrivateUse1) forwards to the backend chosen by
// PYTORCH_BLACKWELL_ALLOC_CONF at first use, so the choice can still be made after this library is loaded.
struct ForwardingAllocator final : public c10::Allocator {
  c10::DataPtr allocate(size_t n) override {
    lazy_init();
    return alloc::get()->allocate(n);
  }
  c10::DeleterFnPtr raw_deleter() const override { return alloc::get()->raw_deleter(); }
  void copy_data(void* dst, const void* src, size_t n) const override { alloc::get()->copy_data(dst, src, n); }
};
ForwardingAllocator g_fwd_alloc;
REGISTER_ALLOCATOR(c10::DeviceType::PrivateUse1, &g_fwd_alloc);

struct Hooks final : public at::PrivateUse1HooksInterface {
  bool isBuilt() const override { return true; }
  bool isAvailable() const override { return device_count() > 0; }
  void init() const override { lazy_init(); }
  bool hasPrimaryContext(c10::DeviceIndex d) const override { return has_primary_context(d); }
  c10::DeviceIndex deviceCount() const override { return device_count(); }
  void setCurrentDevice(c10::DeviceIndex d) const override { set_device(d); }
  c10::DeviceIndex getCurrentDevice() const override { return current_device(); }
  c10::DeviceIndex exchangeDevice(c10::DeviceIndex d) const override { return exchange_device(d); }
  c10::DeviceIndex maybeExchangeDevice(c10::DeviceIndex d) const override { return maybe_exchange_device(d); }
  bool isPinnedPtr(const void* data) const override { return host::is_pinned(data); }
  c10::Allocator* getPinnedMemoryAllocator() const override { return host::pinned_allocator(); }
  c10::Device getDeviceFromPtr(void* data) const override {
    int dev = -1;
    if (alloc::get()->owns(data, &dev)) return make_device(dev);
    cudaPointerAttributes attr{};
    B200_CUDA_CHECK(cudaPointerGetAttributes(&attr, data));
    TORCH_CHECK(attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged,
                "The specified pointer resides on host memory and is not registered with any blackwell device.");
    return make_device(attr.device);
  }
  const at::Generator& getDefaultGenerator(c10::DeviceIndex d) const override { return default_generator(d); }
  at::Generator getNewGenerator(c10::DeviceIndex d) const override { return new_generator(d); }
  void resizePrivateUse1Bytes(const c10::Storage& storage, size_t newsize) const override {
    resize_storage_bytes(storage.unsafeGetStorageImpl(), newsize);
  }
};

c10::once_flag g_init_once;
bool g_initialized = false;

}  // namespace

void register_hooks() {
  static Hooks* h = new Hooks();
  static c10::once_flag once;
  c10::call_once(once, [] { at::RegisterPrivateUse1HooksInterface(h); });
}

void lazy_init() {
  c10::call_once(g_init_once, [] {
    C10_LOG_API_USAGE_ONCE("torch_musa_b200.init");
    auto n = device_count_ensure_non_zero();
    alloc::get()->init(alloc::get()->backend()->device_events ? n : 1);
    if (alloc::config().cpu_unified) host::set_unified_cpu_allocator(true);
    g_initialized = true;
  });
}

bool is_initialized() { return g_initialized; }

void resize_storage_bytes(c10::StorageImpl* storage, size_t newsize) {
  TORCH_CHECK(storage->resizable(), "Trying to resize storage that is not resizable");
  auto* allocator = storage->allocator();
  TORCH_CHECK(allocator != nullptr, "Trying to resize storage without an allocator");
  c10::Device dev = storage->device();
  if (newsize == 0) {
    storage->set_data_ptr_noswap(c10::DataPtr(nullptr, dev));
    storage->set_nbytes(0);
    return;
  }
  DeviceSwitch sw(dev.index());
  c10::DataPtr fresh = allocator->allocate(newsize);
  size_t keep = std::min(storage->nbytes(), newsize);
  if (storage->data_ptr() && keep > 0) {
    B200_CUDA_CHECK(cudaMemcpyAsync(fresh.get(), storage->data(), keep, cudaMemcpyDeviceToDevice,
                                    get_current_stream(dev.index()).stream()));
  }
  storage->set_data_ptr_noswap(std::move(fresh));
  storage->set_nbytes(newsize);
}

}  // namespace b200
