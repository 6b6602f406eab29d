#pragma once

#include "core/Device.h"

#include <c10/core/StorageImpl.h>

namespace b200 {

// Registers the PrivateUse1 hooks object with ATen (idempotent; called at import).
B200_EXPORT void register_hooks();
// First-use initialisation: checks that a GPU exists, sizes the allocator, applies `cpu:unified`.
B200_EXPORT void lazy_init();
B200_EXPORT bool is_initialized();
// Grows/shrinks a device storage, preserving the common prefix (stream-ordered D2D copy).
B200_EXPORT void resize_storage_bytes(c10::StorageImpl* storage, size_t newsize);

}  // namespace b200
