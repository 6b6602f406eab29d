#include "core/Device.h"
#include "core/DeviceAssert.h"

#include <c10/util/CallOnce.h>
#include <c10/util/Logging.h>

#include <array>
#include <atomic>
#include <cstdlib>
#include <mutex>
#include <vector>

namespace b200 {

// Devices on which this process has (as far as the runtime layer knows) created a primary context.
static std::array<std::atomic<bool>, kMaxDevices> g_ctx_touched{};

void check_cuda(cudaError_t err, const char* expr, const char* file, int line) {
  if (err == cudaSuccess) return;
  // Non-sticky errors are cleared so the next call starts clean.
  (void)cudaGetLastError();
  std::string hint;
  if (err == cudaErrorMemoryAllocation) hint = " (out of device memory)";
  TORCH_CHECK(false, "blackwell runtime error: ", cudaGetErrorName(err), ": ", cudaGetErrorString(err), hint,
              "\n  in `", expr, "` at ", file, ":", line,
              "\n  Kernel errors may be reported asynchronously at a later call; set BLACKWELL_LAUNCH_BLOCKING=1 "
              "to localise them.");
}

void warn_cuda(cudaError_t err, const char* expr, const char* file, int line) noexcept {
  if (err == cudaSuccess) return;
  (void)cudaGetLastError();
  try {
    TORCH_WARN("blackwell runtime warning: ", cudaGetErrorName(err), " in `", expr, "` at ", file, ":", line);
  } catch (...) {
  }
}

bool launch_blocking() {
  static const bool v = [] {
    const char* e = std::getenv("BLACKWELL_LAUNCH_BLOCKING");
    return e && std::atoi(e) != 0;
  }();
  return v;
}

void kernel_launch_check(const char* what, cudaStream_t stream) {
  cudaError_t e = cudaGetLastError();
  if (C10_UNLIKELY(e != cudaSuccess)) check_cuda(e, what, __FILE__, __LINE__);
  if (C10_UNLIKELY(launch_blocking())) {
    cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &st) == cudaSuccess && st == cudaStreamCaptureStatusNone) {
      e = cudaStreamSynchronize(stream);
      if (e != cudaSuccess) check_cuda(e, what, __FILE__, __LINE__);
    }
  }
}

c10::DeviceIndex device_count() noexcept {
  static const int n = [] {
    int c = 0;
    cudaError_t e = cudaGetDeviceCount(&c);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return 0;
    }
    return c > kMaxDevices ? kMaxDevices : c;
  }();
  return static_cast<c10::DeviceIndex>(n);
}

c10::DeviceIndex device_count_ensure_non_zero() {
  auto n = device_count();
  TORCH_CHECK(n > 0, "No blackwell (CUDA sm_100) device is visible to this process");
  return n;
}

c10::DeviceIndex current_device() {
  int d = 0;
  B200_CUDA_CHECK(cudaGetDevice(&d));
  return static_cast<c10::DeviceIndex>(d);
}

void set_device(c10::DeviceIndex d) {
  TORCH_CHECK(d >= 0 && d < device_count(), "invalid blackwell device index ", (int)d, " (", (int)device_count(),
              " visible)");
  int cur = -1;
  B200_CUDA_CHECK(cudaGetDevice(&cur));
  if (cur != d) B200_CUDA_CHECK(cudaSetDevice(d));
  g_ctx_touched[d] = true;
}

c10::DeviceIndex exchange_device(c10::DeviceIndex d) {
  int cur = -1;
  B200_CUDA_CHECK(cudaGetDevice(&cur));
  if (d >= 0 && d != cur) B200_CUDA_CHECK(cudaSetDevice(d));
  if (d >= 0 && d < kMaxDevices) g_ctx_touched[d] = true;
  return static_cast<c10::DeviceIndex>(cur);
}

bool has_primary_context(c10::DeviceIndex d) {
  // The runtime API has no primary-context state query; a device counts as initialised once this
  // layer has made it current or queried it (allocator, stream pool and set_device all pass here).
  return d >= 0 && d < kMaxDevices && g_ctx_touched[d].load(std::memory_order_relaxed);
}

c10::DeviceIndex maybe_exchange_device(c10::DeviceIndex d) {
  int cur = -1;
  B200_CUDA_CHECK(cudaGetDevice(&cur));
  if (d < 0 || d == cur) return static_cast<c10::DeviceIndex>(cur);
  if (has_primary_context(d)) B200_CUDA_CHECK(cudaSetDevice(d));
  return static_cast<c10::DeviceIndex>(cur);
}

void device_synchronize() {
  note_implicit_sync("device_synchronize");
  B200_CUDA_CHECK(cudaDeviceSynchronize());
  // kernels that met an out-of-range index (or another recorded condition) report here, as an exception
  int cur = -1;
  if (cudaGetDevice(&cur) == cudaSuccess) check_device_asserts((c10::DeviceIndex)cur);
}

const cudaDeviceProp& device_properties(c10::DeviceIndex d) {
  static std::array<cudaDeviceProp, kMaxDevices> props;
  static std::array<c10::once_flag, kMaxDevices> flags;
  if (d < 0) d = current_device();
  TORCH_CHECK(d < device_count(), "invalid blackwell device index ", (int)d);
  c10::call_once(flags[d], [&] {
    B200_CUDA_CHECK(cudaGetDeviceProperties(&props[d], d));
    g_ctx_touched[d] = true;
  });
  return props[d];
}

namespace {
std::mutex g_peer_mu;
// -1 unknown, 0 no, 1 yes (access enabled)
int8_t g_peer[kMaxDevices][kMaxDevices];
bool g_peer_init = [] {
  for (auto& r : g_peer)
    for (auto& c : r) c = -1;
  return true;
}();
}  // namespace

namespace {
void (*g_peer_hook)(int, int) = nullptr;
}

bool can_access_peer(c10::DeviceIndex a, c10::DeviceIndex b) {
  auto n = device_count();
  TORCH_CHECK(a >= 0 && a < n && b >= 0 && b < n, "invalid peer pair ", (int)a, "->", (int)b);
  if (a == b) return true;
  int ok = 0;
  B200_CUDA_CHECK(cudaDeviceCanAccessPeer(&ok, a, b));
  return ok != 0;
}

bool enable_peer_access(c10::DeviceIndex a, c10::DeviceIndex b) {
  if (a == b) return true;
  std::lock_guard<std::mutex> g(g_peer_mu);
  if (g_peer[a][b] >= 0) return g_peer[a][b] == 1;
  bool ok = can_access_peer(a, b);
  if (ok) {
    DeviceSwitch sw(a);
    cudaError_t e = cudaDeviceEnablePeerAccess(b, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
      (void)cudaGetLastError();
    } else {
      B200_CUDA_CHECK(e);
    }
  }
  g_peer[a][b] = ok ? 1 : 0;
  if (ok && g_peer_hook) g_peer_hook((int)a, (int)b);
  return ok;
}

bool peer_access_enabled(c10::DeviceIndex a, c10::DeviceIndex b) {
  if (a == b) return true;
  if (a < 0 || b < 0 || a >= kMaxDevices || b >= kMaxDevices) return false;
  return g_peer[a][b] == 1;
}

void set_peer_access_hook(void (*hook)(int, int)) { g_peer_hook = hook; }

namespace {
std::atomic<int> g_sync_debug{0};
}
void set_sync_debug_mode(int m) { g_sync_debug = m; }
int sync_debug_mode() { return g_sync_debug; }
void note_implicit_sync(const char* what) {
  int m = g_sync_debug.load(std::memory_order_relaxed);
  if (C10_LIKELY(m == 0)) return;
  if (m == 1) {
    TORCH_WARN("blackwell: host synchronisation in ", what);
  } else {
    TORCH_CHECK(false, "blackwell: host synchronisation in ", what, " while sync-debug mode is 'error'");
  }
}

void memcpy_and_sync(void* dst, const void* src, size_t n, cudaMemcpyKind kind, cudaStream_t s) {
  note_implicit_sync("memcpy_and_sync");
  B200_CUDA_CHECK(cudaMemcpyAsync(dst, src, n, kind, s));
  B200_CUDA_CHECK(cudaStreamSynchronize(s));
}

}  // namespace b200
