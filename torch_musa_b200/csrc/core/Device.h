// Device functions of the "blackwell" backend (PrivateUse1 dispatch key).
//
// The device is CUDA hardware, so a device index here IS the CUDA ordinal and
// "current device" IS the CUDA runtime's current device: our tensors, torch's
// own CUDA tensors and NCCL all agree on it without any translation table.
// Parity: reference torch_musa/csrc/core/MUSAFunctions.h:13-103 (device count
// cache, Get/Set/Exchange/MaybeExchange, sync helpers) and MUSAException.h:7-70
// (checked-call macros, launch-blocking switch).
#pragma once

#include <c10/core/Device.h>
#include <c10/util/Exception.h>
#include <cuda_runtime_api.h>

#include <cstdint>
#include <string>

#define B200_EXPORT __attribute__((visibility("default")))

namespace b200 {

constexpr c10::DeviceType kDeviceType = c10::DeviceType::PrivateUse1;
constexpr const char* kDeviceName = "blackwell";
constexpr int kMaxDevices = 16;

// Throws c10::Error with the CUDA error string; clears the sticky-free error.
B200_EXPORT void check_cuda(cudaError_t err, const char* expr, const char* file, int line);
// Same but only warns (destructors).
B200_EXPORT void warn_cuda(cudaError_t err, const char* expr, const char* file, int line) noexcept;

#define B200_CUDA_CHECK(EXPR)                                   \
  do {                                                          \
    cudaError_t _e = (EXPR);                                    \
    if (C10_UNLIKELY(_e != cudaSuccess))                        \
      ::b200::check_cuda(_e, #EXPR, __FILE__, __LINE__);        \
  } while (0)

#define B200_CUDA_WARN(EXPR)                                    \
  do {                                                          \
    cudaError_t _e = (EXPR);                                    \
    if (C10_UNLIKELY(_e != cudaSuccess))                        \
      ::b200::warn_cuda(_e, #EXPR, __FILE__, __LINE__);         \
  } while (0)

// After a kernel launch: picks up launch-configuration errors and, when
// BLACKWELL_LAUNCH_BLOCKING=1, synchronises so the failing op is the one
// that raises.
B200_EXPORT void kernel_launch_check(const char* what, cudaStream_t stream);
#define B200_KERNEL_LAUNCH_CHECK(STREAM) ::b200::kernel_launch_check(__func__, (STREAM))

// Kernel-library entry points return a cudaError_t as int.
#define B200_KERNEL_CALL(EXPR)                                              \
  do {                                                                      \
    int _e = (EXPR);                                                        \
    if (C10_UNLIKELY(_e != 0))                                              \
      ::b200::check_cuda((cudaError_t)_e, #EXPR, __FILE__, __LINE__);       \
  } while (0)

B200_EXPORT bool launch_blocking();

// 0 when no driver / no GPU is present (CPU-only hosts import fine).
B200_EXPORT c10::DeviceIndex device_count() noexcept;
// Raises a readable error when there is no device.
B200_EXPORT c10::DeviceIndex device_count_ensure_non_zero();
B200_EXPORT c10::DeviceIndex current_device();
B200_EXPORT void set_device(c10::DeviceIndex d);
// Sets `d` current, returns the previous device.
B200_EXPORT c10::DeviceIndex exchange_device(c10::DeviceIndex d);
// Like exchange_device but does not create a context on `d` if the device is
// only being restored and has none yet.
B200_EXPORT c10::DeviceIndex maybe_exchange_device(c10::DeviceIndex d);
B200_EXPORT void device_synchronize();
B200_EXPORT bool has_primary_context(c10::DeviceIndex d);
B200_EXPORT const cudaDeviceProp& device_properties(c10::DeviceIndex d);
B200_EXPORT bool can_access_peer(c10::DeviceIndex a, c10::DeviceIndex b);
// Lazily enables peer access a->b once; returns whether access is possible.
B200_EXPORT bool enable_peer_access(c10::DeviceIndex a, c10::DeviceIndex b);
// True once enable_peer_access(a, b) has succeeded (a reads/writes b's memory); never calls the driver.
B200_EXPORT bool peer_access_enabled(c10::DeviceIndex a, c10::DeviceIndex b);
// Called as hook(a, b) after a gains access to b: memory mapped outside cudaMalloc needs an explicit grant.
B200_EXPORT void set_peer_access_hook(void (*hook)(int a, int b));

// Sync-debug mode: 0 off, 1 warn, 2 error on implicit host synchronisation.
B200_EXPORT void set_sync_debug_mode(int m);
B200_EXPORT int sync_debug_mode();
B200_EXPORT void note_implicit_sync(const char* what);

// memcpy + stream sync with the sync-debug bookkeeping.
B200_EXPORT void memcpy_and_sync(void* dst, const void* src, size_t n, cudaMemcpyKind kind, cudaStream_t s);

inline c10::Device make_device(c10::DeviceIndex i) { return c10::Device(kDeviceType, i); }

// RAII device switch that restores on scope exit.
struct B200_EXPORT DeviceSwitch {
  explicit DeviceSwitch(c10::DeviceIndex d) {
    if (d >= 0) { prev_ = exchange_device(d); armed_ = (prev_ != d); }
  }
  ~DeviceSwitch() { if (armed_) cudaSetDevice(prev_); }
  DeviceSwitch(const DeviceSwitch&) = delete;
  DeviceSwitch& operator=(const DeviceSwitch&) = delete;
 private:
  c10::DeviceIndex prev_ = -1;
  bool armed_ = false;
};

}  // namespace b200
