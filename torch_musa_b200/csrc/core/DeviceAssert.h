// Device-side assertions without traps.  A kernel that meets a condition it must not continue through (an index
// out of range, a wait that ran out) records a code in a host-mapped word of its device and carries on with a safe
// value; the host checks the word at every explicit synchronisation and raises a normal exception, so the context
// survives.  Each kernel family registers a short description of its codes.
// Parity: reference torch_musa/csrc/core/MUSAException.h (device-side assertion registry, inert there: the
// reference compiles its launch registry out); trapping asserts are deliberately not used here.
#pragma once

#include "core/Device.h"

#include <string>

namespace b200 {

enum DeviceAssertCode : int { kAssertNone = 0, kAssertIndexOutOfRange = 1 };

// Device pointer of the assertion word of `device` (created on first use; one int per device).
B200_EXPORT int* device_assert_word(c10::DeviceIndex device);
// Reads and clears the word; returns the code that was recorded (0: none).
B200_EXPORT int take_device_assert(c10::DeviceIndex device);
// take_device_assert + TORCH_CHECK with the registered description.
B200_EXPORT void check_device_asserts(c10::DeviceIndex device);
B200_EXPORT void register_device_assert(int code, const std::string& what);

}  // namespace b200
