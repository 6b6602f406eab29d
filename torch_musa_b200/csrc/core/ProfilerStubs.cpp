// Profiler stubs for the blackwell device: what the legacy autograd profiler (`use_device="blackwell"`) calls to
// time operators on the device -- record an event on the current stream, measure elapsed time between two events,
// run a callback on every device, synchronise.  NVTX-style marks and ranges go to torch's own NVTX path and are
// no-ops here.  (Kineto/CUPTI traces need none of this: the kernels are CUDA kernels.)
// Parity: reference torch_musa/csrc/profiler/stubs.cpp:39-102.
#include <nvtx3/nvToolsExt.h>
#include "core/Device.h"
#include "core/Stream.h"

#include <c10/util/ApproximateClock.h>
#include <torch/csrc/profiler/stubs/base.h>

#include <cuda_runtime_api.h>

namespace b200 {
namespace {

using torch::profiler::impl::ProfilerVoidEventStub;

struct EventHolder {
  cudaEvent_t ev = nullptr;
  ~EventHolder() {
    if (ev) cudaEventDestroy(ev);
  }
};

struct BlackwellProfilerStubs : public torch::profiler::impl::ProfilerStubs {
  void record(c10::DeviceIndex* device, ProfilerVoidEventStub* event, int64_t* cpu_ns) const override {
    int dev = 0;
    B200_CUDA_CHECK(cudaGetDevice(&dev));
    if (device) *device = (c10::DeviceIndex)dev;
    auto holder = std::make_shared<EventHolder>();
    B200_CUDA_CHECK(cudaEventCreate(&holder->ev));
    cudaStream_t stream = get_current_stream((c10::DeviceIndex)dev).stream();
    if (cpu_ns) *cpu_ns = c10::getTime();
    B200_CUDA_CHECK(cudaEventRecord(holder->ev, stream));
    *event = std::static_pointer_cast<void>(holder);
  }

  float elapsed(const ProfilerVoidEventStub* a, const ProfilerVoidEventStub* b) const override {
    auto* ea = static_cast<EventHolder*>(a->get());
    auto* eb = static_cast<EventHolder*>(b->get());
    B200_CUDA_CHECK(cudaEventSynchronize(ea->ev));
    B200_CUDA_CHECK(cudaEventSynchronize(eb->ev));
    float ms = 0.f;
    B200_CUDA_CHECK(cudaEventElapsedTime(&ms, ea->ev, eb->ev));
    return ms * 1000.f;  // microseconds
  }

  // NVTX (header-only v3: the calls are no-ops until a tool injects its library), so that ranges emitted through
  // torch.autograd.profiler.emit_nvtx / record_function show up on the timeline of an attached profiler
  void mark(const char* name) const override { nvtxMarkA(name ? name : ""); }
  void rangePush(const char* name) const override { nvtxRangePushA(name ? name : ""); }
  void rangePop() const override { nvtxRangePop(); }
  bool enabled() const override { return true; }

  void onEachDevice(std::function<void(int)> op) const override {
    int cur = 0, n = 0;
    B200_CUDA_CHECK(cudaGetDevice(&cur));
    B200_CUDA_CHECK(cudaGetDeviceCount(&n));
    for (int i = 0; i < n; ++i) {
      B200_CUDA_CHECK(cudaSetDevice(i));
      op(i);
    }
    B200_CUDA_CHECK(cudaSetDevice(cur));
  }

  void synchronize() const override { B200_CUDA_CHECK(cudaDeviceSynchronize()); }
};

struct RegisterStubs {
  RegisterStubs() {
    static BlackwellProfilerStubs stubs;
    torch::profiler::impl::registerPrivateUse1Methods(&stubs);
  }
};
RegisterStubs g_register_stubs;

}  // namespace
}  // namespace b200
