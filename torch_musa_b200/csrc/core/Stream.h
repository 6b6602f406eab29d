// Stream pool, thread-local current streams and RAII events.
//
// A blackwell stream is a cudaStream_t wrapped in a c10::Stream whose id encodes
// where it came from:
//   id == 0                       the device's default (legacy NULL) stream
//   id odd : ((prio*32+slot)<<1)|1 a pool stream (32 per priority level, round-robin)
//   id even, != 0                 an external cudaStream_t handed in by the user
// Pool streams are created lazily per device and never destroyed (process
// lifetime), like every PyTorch backend.  Parity: reference
// torch_musa/csrc/core/MUSAStream.h:19-176, MUSAStream.cpp:17-255 (pool of 32 x
// priorities, id packing, external streams) and MUSAEvent.h:33-240.
#pragma once

#include <optional>
#include <utility>
#include <vector>

#include "core/Device.h"

#include <c10/core/Stream.h>

namespace b200 {

constexpr int kStreamsPerPool = 32;
constexpr int kMaxPriorities = 4;

class B200_EXPORT Stream {
 public:
  explicit Stream(c10::Stream s) : s_(s) {
    TORCH_CHECK(s.device_type() == kDeviceType, "not a blackwell stream");
  }
  c10::Stream unwrap() const { return s_; }
  operator c10::Stream() const { return s_; }
  c10::DeviceIndex device_index() const { return s_.device_index(); }
  c10::StreamId id() const { return s_.id(); }
  cudaStream_t stream() const;
  operator cudaStream_t() const { return stream(); }
  bool query() const;
  void synchronize() const;
  int priority() const;
  bool operator==(const Stream& o) const { return s_ == o.s_; }
  bool operator!=(const Stream& o) const { return !(s_ == o.s_); }

 private:
  c10::Stream s_;
};

// Number of usable priority levels (<= kMaxPriorities) and CUDA's [least, greatest] range.
B200_EXPORT int num_priorities();
B200_EXPORT void priority_range(int* least, int* greatest);

// priority: 0 = default, negative = higher priority (clamped to what the device offers).
B200_EXPORT Stream get_stream_from_pool(int priority = 0, c10::DeviceIndex device = -1);
B200_EXPORT Stream get_stream_from_pool(bool high_priority, c10::DeviceIndex device);
B200_EXPORT Stream get_stream_from_external(cudaStream_t ext, c10::DeviceIndex device);
B200_EXPORT Stream get_default_stream(c10::DeviceIndex device = -1);
B200_EXPORT Stream get_current_stream(c10::DeviceIndex device = -1);
B200_EXPORT void set_current_stream(Stream s);
B200_EXPORT cudaStream_t stream_from_c10(c10::Stream s);

// --------------------------------------------------------------------------
// Event: lazily created on first record, bound to the recording device.
class B200_EXPORT Event {
 public:
  Event() = default;
  explicit Event(unsigned flags) : flags_(flags) {}
  ~Event();
  Event(const Event&) = delete;
  Event& operator=(const Event&) = delete;
  Event(Event&& o) noexcept { move_from(std::move(o)); }
  Event& operator=(Event&& o) noexcept {
    if (this != &o) { destroy(); move_from(std::move(o)); }
    return *this;
  }

  bool is_created() const { return created_; }
  c10::DeviceIndex device_index() const { return device_; }
  cudaEvent_t event() const { return ev_; }
  bool query() const;
  void record();
  void record(const Stream& s);
  void record_once(const Stream& s);
  void block(const Stream& s) const;   // make `s` wait for this event
  void synchronize() const;
  float elapsed_ms(const Event& later) const;
  // Inter-process handle (events created with cudaEventInterprocess|DisableTiming).
  void ipc_handle(cudaIpcEventHandle_t* out);
  static Event from_ipc_handle(c10::DeviceIndex device, const cudaIpcEventHandle_t* h);

 private:
  void create(c10::DeviceIndex d);
  void destroy() noexcept;
  void move_from(Event&& o) noexcept;
  unsigned flags_ = cudaEventDisableTiming;
  bool created_ = false;
  bool recorded_ = false;
  c10::DeviceIndex device_ = -1;
  cudaEvent_t ev_ = nullptr;
};

// (reused, newly created) event counts of the event cache
B200_EXPORT std::pair<int64_t, int64_t> event_cache_stats();

// RAII: make `s` the current stream of its device (and that device current).
struct B200_EXPORT StreamGuard {
  explicit StreamGuard(Stream s);
  ~StreamGuard();
  StreamGuard(const StreamGuard&) = delete;
  StreamGuard& operator=(const StreamGuard&) = delete;
 private:
  c10::DeviceIndex prev_device_;
  Stream prev_stream_;
};

// A StreamGuard that may stay empty: reset_stream() arms it (or moves it to another stream), the destructor
// restores whatever was current before the first arming.
// Parity: reference torch_musa/csrc/core/MUSAGuard.h (OptionalMUSAStreamGuard, MUSAMultiStreamGuard).
class OptionalStreamGuard {
 public:
  OptionalStreamGuard() = default;
  explicit OptionalStreamGuard(Stream s) { reset_stream(s); }
  explicit OptionalStreamGuard(std::optional<Stream> s) {
    if (s.has_value()) reset_stream(*s);
  }
  void reset_stream(Stream s) {
    guard_.reset();  // restore first: the guard below must remember the ORIGINAL stream of its device
    guard_.emplace(s);
  }
  void reset() { guard_.reset(); }
  bool armed() const { return guard_.has_value(); }

 private:
  std::optional<StreamGuard> guard_;
};

// Sets the current stream of several devices at once (at most one stream per device) and restores them all.
class MultiStreamGuard {
 public:
  explicit MultiStreamGuard(const std::vector<Stream>& streams) {
    prev_.reserve(streams.size());
    for (const Stream& s : streams) {
      prev_.push_back(get_current_stream(s.device_index()));
      set_current_stream(s);
    }
  }
  ~MultiStreamGuard() {
    for (auto it = prev_.rbegin(); it != prev_.rend(); ++it) set_current_stream(*it);
  }
  MultiStreamGuard(const MultiStreamGuard&) = delete;
  MultiStreamGuard& operator=(const MultiStreamGuard&) = delete;

 private:
  std::vector<Stream> prev_;
};

}  // namespace b200
