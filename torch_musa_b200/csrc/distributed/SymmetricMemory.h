// Peer-mapped ("symmetric") memory for one process group on one device.
//
// Every rank allocates an arena of the same size plus a small signal pad, exports both
// with CUDA IPC handles through the group's store and maps every peer's pair into its
// own address space.  The backend's collective kernels then load/store peer HBM over
// NVLink directly.  The arena is split into two halves used by alternating calls
// (double buffering removes the trailing barrier of pull-style collectives); epochs
// handed out by next_epoch() advance identically on all ranks because all ranks issue
// the same collectives in the same order.
// Parity: the reference's VMM handle-sharing skeleton (reference
// torch_musa/csrc/core/MUSACachingAllocator.cpp:189-392) and its external ce_comm hook
// (torch_musa/distributed/_composable/fsdp/custom_overlap_patch.py:46-116).
#pragma once

#include "core/Device.h"
#include "kernels/b200_kernels.h"

#include <ATen/core/Tensor.h>
#include <torch/csrc/distributed/c10d/Store.hpp>

#include <string>
#include <vector>

namespace b200 {
namespace dist {

class B200_EXPORT SymmetricMemory {
 public:
  SymmetricMemory(c10::intrusive_ptr<c10d::Store> store, const std::string& key, int rank, int world,
                  c10::DeviceIndex device, size_t half_bytes);
  ~SymmetricMemory();
  SymmetricMemory(const SymmetricMemory&) = delete;

  bool ok() const { return ok_; }
  const std::string& why_not() const { return why_not_; }
  int rank() const { return rank_; }
  int world() const { return world_; }
  size_t half_bytes() const { return half_; }
  const b200_symm_t* desc() const { return &desc_; }
  // Epoch for the next collective (advances by 2) and the arena half that call must use.
  uint32_t next_epoch(int64_t* half_offset);
  // Non-zero if any kernel on this arena gave up on a bounded wait (cleared by the read).
  int take_status();
  // Same word without clearing it.
  int peek_status() const { return status_host_ ? *(volatile int*)status_host_ : 0; }
  // A tensor view over the local arena (byte offset from the arena base).
  at::Tensor local_tensor(int64_t byte_offset, at::IntArrayRef sizes, at::ScalarType dtype);
  void* peer_base(int r) const { return desc_.bufs[r]; }

 private:
  c10::intrusive_ptr<c10d::Store> store_;
  int rank_, world_;
  c10::DeviceIndex device_;
  size_t half_;
  bool ok_ = false;
  std::string why_not_;
  void* arena_ = nullptr;
  void* pad_ = nullptr;
  int* status_host_ = nullptr;
  std::vector<void*> opened_;
  b200_symm_t desc_{};
  uint32_t epoch_ = 2;
};

}  // namespace dist
}  // namespace b200
