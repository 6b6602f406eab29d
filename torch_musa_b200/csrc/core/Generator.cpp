#include "core/Generator.h"

#include <ATen/Functions.h>
#include <ATen/Utils.h>
#include <c10/util/CallOnce.h>

#include <cstring>
#include <deque>
#include <random>

namespace b200 {

GeneratorImpl::GeneratorImpl(c10::DeviceIndex device)
    : c10::GeneratorImpl(make_device(device), c10::DispatchKeySet(c10::DispatchKey::PrivateUse1)) {}

void GeneratorImpl::set_current_seed(uint64_t seed) {
  TORCH_CHECK(!capturing_, "cannot reseed a generator while a graph capture that uses it is under way");
  seed_ = seed;
  offset_ = 0;
}
void GeneratorImpl::set_offset(uint64_t offset) {
  TORCH_CHECK(!capturing_, "cannot set the offset of a generator during graph capture");
  TORCH_CHECK(offset % 4 == 0, "philox offset must be a multiple of 4");
  offset_ = offset;
}
uint64_t GeneratorImpl::get_offset() const { return offset_; }
uint64_t GeneratorImpl::current_seed() const { return seed_; }
uint64_t GeneratorImpl::seed() {
  std::random_device rd;
  uint64_t s = ((uint64_t)rd() << 32) | rd();
  set_current_seed(s);
  return s;
}

// State layout (16 bytes, little endian): seed, offset -- the same two words torch's CUDA generator saves,
// so an RNG state saved on one backend can be loaded on the other.
c10::intrusive_ptr<c10::TensorImpl> GeneratorImpl::get_state() const {
  auto t = at::empty({16}, at::TensorOptions().dtype(at::kByte).device(at::kCPU));
  auto* p = t.data_ptr<uint8_t>();
  std::memcpy(p, &seed_, 8);
  int64_t off = (int64_t)offset_;
  std::memcpy(p + 8, &off, 8);
  return t.getIntrusivePtr();
}

void GeneratorImpl::set_state(const c10::TensorImpl& st) {
  at::detail::check_rng_state(st);
  TORCH_CHECK(st.numel() == 16, "blackwell RNG state must be 16 bytes, got ", st.numel());
  const auto* p = static_cast<const uint8_t*>(st.data());
  uint64_t s;
  int64_t off;
  std::memcpy(&s, p, 8);
  std::memcpy(&off, p + 8, 8);
  set_current_seed(s);
  set_offset((uint64_t)off);
}

PhiloxArgs GeneratorImpl::philox_args(uint64_t increment) {
  increment = (increment + 3) / 4 * 4;
  PhiloxArgs a{};
  if (capturing_) {
    a.seed_ptr = seed_dev_;
    a.offset_ptr = offset_dev_;
    a.offset_intragraph = offset_intragraph_;
    a.captured = 1;
    offset_intragraph_ += increment;
  } else {
    a.seed = seed_;
    a.offset = offset_;
    offset_ += increment;
  }
  return a;
}

void GeneratorImpl::capture_prologue(int64_t* seed_dev, int64_t* offset_dev) {
  capturing_ = true;
  seed_dev_ = seed_dev;
  offset_dev_ = offset_dev;
  offset_intragraph_ = 0;
}

uint64_t GeneratorImpl::capture_epilogue() {
  capturing_ = false;
  return offset_intragraph_;
}

GeneratorImpl* GeneratorImpl::clone_impl() const {
  auto* g = new GeneratorImpl(device().index());
  g->seed_ = seed_;
  g->offset_ = offset_;
  return g;
}

const at::Generator& default_generator(c10::DeviceIndex device) {
  static std::deque<at::Generator> gens;
  static c10::once_flag once;
  c10::call_once(once, [] {
    int n = std::max<int>(device_count(), 1);
    for (int i = 0; i < n; ++i) {
      gens.push_back(at::make_generator<GeneratorImpl>((c10::DeviceIndex)i));
      gens.back().seed();
    }
  });
  if (device < 0) device = device_count() > 0 ? current_device() : 0;
  TORCH_CHECK(device < (int)gens.size(), "invalid blackwell device index ", (int)device);
  return gens[device];
}

at::Generator new_generator(c10::DeviceIndex device) {
  if (device < 0) device = device_count() > 0 ? current_device() : 0;
  return at::make_generator<GeneratorImpl>(device);
}

}  // namespace b200
