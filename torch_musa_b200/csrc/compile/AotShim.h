// C ABI through which ahead-of-time compiled code (a wrapper compiled as plain C or against another C++ runtime)
// manages this backend's device and stream state without seeing any C++ type of it: opaque guard handles, the
// current stream of a device, and the device-type code to put into tensor handles.  Every call returns 0 on success
// and 1 on failure; the message of the calling thread's last failure is available from b200_shim_last_error().
// The `aoti_torch_*_blackwell*` names are the ones a generated Inductor C++ wrapper asks a device for.
// C++ users get RAII wrappers below the C declarations.
//
// Parity: reference torch_musa/csrc/inductor/aoti_torch/shim_musa.cpp:9-61 and aoti_runtime/utils_musa.h:24-54.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t B200ShimError;
typedef struct B200DeviceGuardOpaque* B200DeviceGuardHandle;
typedef struct B200StreamGuardOpaque* B200StreamGuardHandle;

#define B200_SHIM_API __attribute__((visibility("default")))

B200_SHIM_API B200ShimError aoti_torch_create_blackwell_guard(int32_t device_index, B200DeviceGuardHandle* ret_guard);
B200_SHIM_API B200ShimError aoti_torch_delete_blackwell_guard(B200DeviceGuardHandle guard);
B200_SHIM_API B200ShimError aoti_torch_blackwell_guard_set_index(B200DeviceGuardHandle guard, int32_t device_index);
/* `stream` is a raw cudaStream_t; it becomes the current stream of `device_index` until the guard is deleted */
B200_SHIM_API B200ShimError aoti_torch_create_blackwell_stream_guard(void* stream, int32_t device_index,
                                                                     B200StreamGuardHandle* ret_guard);
B200_SHIM_API B200ShimError aoti_torch_delete_blackwell_stream_guard(B200StreamGuardHandle guard);
B200_SHIM_API B200ShimError aoti_torch_get_current_blackwell_stream(int32_t device_index, void** ret_stream);
B200_SHIM_API int32_t aoti_torch_device_type_blackwell(void);
B200_SHIM_API const char* b200_shim_last_error(void);

#ifdef __cplusplus
}  // extern "C"

#include <memory>
#include <stdexcept>

namespace b200 {
namespace aot {

inline void shim_check(B200ShimError e) {
  if (e != 0) throw std::runtime_error(b200_shim_last_error());
}

// Makes a device current for a scope (and can be re-pointed inside it).
class DeviceGuard {
 public:
  explicit DeviceGuard(int32_t device_index) : h_(nullptr, &aoti_torch_delete_blackwell_guard) {
    B200DeviceGuardHandle p = nullptr;
    shim_check(aoti_torch_create_blackwell_guard(device_index, &p));
    h_.reset(p);
  }
  void set_index(int32_t device_index) { shim_check(aoti_torch_blackwell_guard_set_index(h_.get(), device_index)); }

 private:
  std::unique_ptr<B200DeviceGuardOpaque, B200ShimError (*)(B200DeviceGuardHandle)> h_;
};

// Makes a raw stream the current stream of its device for a scope.
class StreamGuard {
 public:
  StreamGuard(void* raw_stream, int32_t device_index) : h_(nullptr, &aoti_torch_delete_blackwell_stream_guard) {
    B200StreamGuardHandle p = nullptr;
    shim_check(aoti_torch_create_blackwell_stream_guard(raw_stream, device_index, &p));
    h_.reset(p);
  }

 private:
  std::unique_ptr<B200StreamGuardOpaque, B200ShimError (*)(B200StreamGuardHandle)> h_;
};

}  // namespace aot
}  // namespace b200
#endif
