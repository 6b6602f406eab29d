// Implementation of the C ABI of AotShim.h over the runtime's own guards.
#include "compile/AotShim.h"

#include "core/Device.h"
#include "core/Stream.h"

#include <c10/core/DeviceType.h>

#include <exception>
#include <memory>
#include <optional>
#include <string>

namespace {

thread_local std::string g_last_error;

template <typename F>
B200ShimError guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_last_error = e.what();
  } catch (...) {
    g_last_error = "unknown failure";
  }
  return 1;
}

// A re-pointable device switch: restores the device that was current when it was created.
struct DeviceGuardImpl {
  explicit DeviceGuardImpl(int32_t d) { sw.emplace((c10::DeviceIndex)d); }
  void set(int32_t d) {
    sw.reset();           // back to the original device first, so that the original is what gets restored in the end
    sw.emplace((c10::DeviceIndex)d);
  }
  std::optional<b200::DeviceSwitch> sw;
};

}  // namespace

extern "C" {

B200ShimError aoti_torch_create_blackwell_guard(int32_t device_index, B200DeviceGuardHandle* ret_guard) {
  return guarded([&] {
    TORCH_CHECK(ret_guard != nullptr, "null result pointer");
    TORCH_CHECK(device_index >= 0 && device_index < b200::device_count(), "device index ", device_index, " out of range");
    *ret_guard = reinterpret_cast<B200DeviceGuardHandle>(new DeviceGuardImpl(device_index));
  });
}

B200ShimError aoti_torch_delete_blackwell_guard(B200DeviceGuardHandle guard) {
  return guarded([&] { delete reinterpret_cast<DeviceGuardImpl*>(guard); });
}

B200ShimError aoti_torch_blackwell_guard_set_index(B200DeviceGuardHandle guard, int32_t device_index) {
  return guarded([&] {
    TORCH_CHECK(guard != nullptr, "null guard");
    TORCH_CHECK(device_index >= 0 && device_index < b200::device_count(), "device index ", device_index, " out of range");
    reinterpret_cast<DeviceGuardImpl*>(guard)->set(device_index);
  });
}

B200ShimError aoti_torch_create_blackwell_stream_guard(void* stream, int32_t device_index, B200StreamGuardHandle* ret_guard) {
  return guarded([&] {
    TORCH_CHECK(ret_guard != nullptr, "null result pointer");
    TORCH_CHECK(device_index >= 0 && device_index < b200::device_count(), "device index ", device_index, " out of range");
    auto s = b200::get_stream_from_external(static_cast<cudaStream_t>(stream), (c10::DeviceIndex)device_index);
    *ret_guard = reinterpret_cast<B200StreamGuardHandle>(new b200::StreamGuard(s));
  });
}

B200ShimError aoti_torch_delete_blackwell_stream_guard(B200StreamGuardHandle guard) {
  return guarded([&] { delete reinterpret_cast<b200::StreamGuard*>(guard); });
}

B200ShimError aoti_torch_get_current_blackwell_stream(int32_t device_index, void** ret_stream) {
  return guarded([&] {
    TORCH_CHECK(ret_stream != nullptr, "null result pointer");
    TORCH_CHECK(device_index >= 0 && device_index < b200::device_count(), "device index ", device_index, " out of range");
    *ret_stream = static_cast<void*>(b200::get_current_stream((c10::DeviceIndex)device_index).stream());
  });
}

int32_t aoti_torch_device_type_blackwell(void) { return (int32_t)c10::DeviceType::PrivateUse1; }

const char* b200_shim_last_error(void) { return g_last_error.c_str(); }

}  // extern "C"
