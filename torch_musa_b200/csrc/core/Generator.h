// Philox-4x32 generator state for the blackwell device.
//
// Kernels that need randomness (dropout, uniform_, normal_, bernoulli_) receive
// a PhiloxArgs by value.  Outside graph capture it carries the seed and the
// running offset as immediates; during capture it carries device pointers to a
// seed word and an "offset at replay" word plus the offset consumed so far inside
// the graph, and every replay bumps the extragraph offset by the graph's total.
// Parity: reference torch_musa/csrc/aten/musa/MUSAGeneratorImpl.h:97-163.
#pragma once

#include "core/Device.h"

#include <ATen/core/Generator.h>
#include <c10/core/GeneratorImpl.h>

namespace b200 {

struct PhiloxArgs {
  uint64_t seed;
  uint64_t offset;
  const int64_t* seed_ptr;      // non-null only while capturing
  const int64_t* offset_ptr;    // non-null only while capturing
  uint64_t offset_intragraph;
  int captured;
};

struct B200_EXPORT GeneratorImpl final : public c10::GeneratorImpl {
  explicit GeneratorImpl(c10::DeviceIndex device);
  ~GeneratorImpl() override = default;

  void set_current_seed(uint64_t seed) override;
  void set_offset(uint64_t offset) override;
  uint64_t get_offset() const override;
  uint64_t current_seed() const override;
  uint64_t seed() override;
  void set_state(const c10::TensorImpl& new_state) override;
  c10::intrusive_ptr<c10::TensorImpl> get_state() const override;
  static c10::DeviceType device_type() { return kDeviceType; }

  // Reserves `increment` Philox counters (rounded up to a multiple of 4) and returns kernel arguments.
  PhiloxArgs philox_args(uint64_t increment);

  // Graph capture protocol.
  void capture_prologue(int64_t* seed_dev, int64_t* offset_dev);
  uint64_t capture_epilogue();  // returns the whole-graph increment
  void advance_after_replay(uint64_t whole_graph_increment) { offset_ += whole_graph_increment; }
  bool capturing() const { return capturing_; }

 private:
  GeneratorImpl* clone_impl() const override;
  uint64_t seed_ = 67280421310721ull;  // torch's default seed
  uint64_t offset_ = 0;
  bool capturing_ = false;
  int64_t* seed_dev_ = nullptr;
  int64_t* offset_dev_ = nullptr;
  uint64_t offset_intragraph_ = 0;
};

B200_EXPORT const at::Generator& default_generator(c10::DeviceIndex device = -1);
B200_EXPORT at::Generator new_generator(c10::DeviceIndex device = -1);

}  // namespace b200
