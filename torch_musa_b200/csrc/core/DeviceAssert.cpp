#include "core/DeviceAssert.h"

#include <array>
#include <map>
#include <mutex>

namespace b200 {
namespace {
struct Word {
  int* host = nullptr;
  int* dev = nullptr;
};
std::array<Word, kMaxDevices> g_words;
std::mutex g_mu;
std::map<int, std::string>& table() {
  static std::map<int, std::string> t{{kAssertIndexOutOfRange, "index out of range in a device kernel (the access was clamped)"}};
  return t;
}
}  // namespace

int* device_assert_word(c10::DeviceIndex device) {
  std::lock_guard<std::mutex> g(g_mu);
  Word& w = g_words.at(device);
  if (!w.dev) {
    DeviceSwitch sw(device);
    B200_CUDA_CHECK(cudaHostAlloc((void**)&w.host, sizeof(int), cudaHostAllocMapped));
    *w.host = 0;
    B200_CUDA_CHECK(cudaHostGetDevicePointer((void**)&w.dev, w.host, 0));
  }
  return w.dev;
}

int take_device_assert(c10::DeviceIndex device) {
  std::lock_guard<std::mutex> g(g_mu);
  if (device < 0 || device >= (c10::DeviceIndex)g_words.size()) return 0;
  Word& w = g_words[device];
  if (!w.host) return 0;
  const int v = *(volatile int*)w.host;
  if (v) *(volatile int*)w.host = 0;
  return v;
}

void register_device_assert(int code, const std::string& what) {
  std::lock_guard<std::mutex> g(g_mu);
  table()[code] = what;
}

void check_device_asserts(c10::DeviceIndex device) {
  const int v = take_device_assert(device);
  if (!v) return;
  std::string what;
  {
    std::lock_guard<std::mutex> g(g_mu);
    auto it = table().find(v);
    what = it != table().end() ? it->second : "device-side assertion " + std::to_string(v);
  }
  TORCH_CHECK_INDEX(false, "blackwell device ", (int)device, ": ", what);
}

}  // namespace b200
