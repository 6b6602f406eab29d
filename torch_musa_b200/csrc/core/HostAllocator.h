// Caching pinned-host allocator and the unified-memory CPU allocator.
//
// Pinned blocks come from cudaHostAlloc (or malloc + cudaHostRegister when
// `pinned_use_host_register` is set), are bucketed by power-of-two size, and a
// freed block is only reused after every stream that read or wrote it (H2D /
// D2H copies call record_event) has passed the recorded event.
//
// The "UMA CPU allocator" hands out cudaMallocManaged memory for *CPU* tensors
// so that a checkpoint loaded with map_location=<device> can be retagged to
// the device without a second allocation or a copy.
//
// Parity: reference torch_musa/csrc/core/CachingHostAllocator.cpp:18-198,
// UMACPUAllocator.cpp:10-40.
#pragma once

#include "core/Device.h"
#include "core/Stream.h"

#include <c10/core/Allocator.h>

namespace b200 {
namespace host {

struct HostStats {
  int64_t allocations = 0, frees = 0, cached_blocks = 0, cached_bytes = 0, active_blocks = 0, active_bytes = 0,
          device_allocs = 0, reuse_hits = 0, events_pending = 0;
};

B200_EXPORT c10::Allocator* pinned_allocator();
// Notes that `stream` uses the pinned block behind `ptr` (any interior pointer). Returns false if not ours.
B200_EXPORT bool record_event(const void* ptr, void* ctx, const Stream& stream);
B200_EXPORT bool is_pinned(const void* ptr);
B200_EXPORT void empty_cache();
B200_EXPORT HostStats stats();

// Managed-memory allocator usable as the CPU allocator.
B200_EXPORT c10::Allocator* unified_cpu_allocator();
B200_EXPORT void set_unified_cpu_allocator(bool on);
B200_EXPORT bool unified_cpu_allocator_enabled();
B200_EXPORT bool is_managed_ptr(const void* p);

}  // namespace host
}  // namespace b200
