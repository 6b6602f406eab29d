#include "distributed/SymmetricMemory.h"

#include "core/Backend.h"

#include <ATen/Functions.h>
#include <unistd.h>

#include <cstring>

namespace b200 {
namespace dist {

namespace {
struct Exported {
  cudaIpcMemHandle_t arena, pad;
  int64_t pid;
  int32_t device;
  char host[64];
};
}  // namespace

SymmetricMemory::SymmetricMemory(c10::intrusive_ptr<c10d::Store> store, const std::string& key, int rank, int world,
                                 c10::DeviceIndex device, size_t half_bytes)
    : store_(std::move(store)), rank_(rank), world_(world), device_(device), half_(half_bytes) {
  if (world_ > b200_comm_max_world()) {
    why_not_ = "group larger than the kernels' peer table";
    return;
  }
  DeviceSwitch sw(device_);
  const size_t pad_bytes = b200_comm_signal_bytes();
  cudaError_t e = cudaMalloc(&arena_, 2 * half_);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    why_not_ = std::string("arena allocation failed: ") + cudaGetErrorString(e);
    arena_ = nullptr;
  }
  if (arena_) {
    B200_CUDA_CHECK(cudaMalloc(&pad_, pad_bytes));
    B200_CUDA_CHECK(cudaMemset(pad_, 0, pad_bytes));
    B200_CUDA_CHECK(cudaHostAlloc((void**)&status_host_, sizeof(int), cudaHostAllocMapped));
    *status_host_ = 0;
    B200_CUDA_CHECK(cudaDeviceSynchronize());
  }
  // Every rank publishes a record (even a failed one) so that nobody blocks on a missing key.
  Exported mine{};
  mine.pid = arena_ ? (int64_t)getpid() : -1;
  mine.device = device_;
  gethostname(mine.host, sizeof(mine.host) - 1);
  if (arena_ && world_ > 1) {
    B200_CUDA_CHECK(cudaIpcGetMemHandle(&mine.arena, arena_));
    B200_CUDA_CHECK(cudaIpcGetMemHandle(&mine.pad, pad_));
  }
  std::vector<Exported> all(world_);
  if (world_ > 1) {
    std::vector<uint8_t> bytes(sizeof(Exported));
    std::memcpy(bytes.data(), &mine, sizeof(Exported));
    store_->set(key + "/" + std::to_string(rank_), bytes);
    for (int r = 0; r < world_; ++r) {
      auto v = store_->get(key + "/" + std::to_string(r));
      TORCH_CHECK(v.size() == sizeof(Exported), "symmetric memory: malformed peer record");
      std::memcpy(&all[r], v.data(), sizeof(Exported));
    }
  } else {
    all[0] = mine;
  }
  bool usable = true;
  for (int r = 0; r < world_; ++r) {
    if (all[r].pid < 0) { usable = false; why_not_ = "a peer could not allocate its arena"; }
    if (std::strncmp(all[r].host, mine.host, sizeof(mine.host)) != 0) {
      usable = false;
      why_not_ = "ranks span several hosts (peer mapping is intra-node)";
    }
  }
  desc_.rank = rank_;
  desc_.world = world_;
  if (usable) {
    for (int r = 0; r < world_ && usable; ++r) {
      if (r == rank_) {
        desc_.bufs[r] = arena_;
        desc_.sigs[r] = static_cast<uint32_t*>(pad_);
        continue;
      }
      void *pa = nullptr, *pp = nullptr;
      cudaError_t e1 = cudaIpcOpenMemHandle(&pa, all[r].arena, cudaIpcMemLazyEnablePeerAccess);
      cudaError_t e2 = e1 == cudaSuccess ? cudaIpcOpenMemHandle(&pp, all[r].pad, cudaIpcMemLazyEnablePeerAccess) : e1;
      if (e1 != cudaSuccess || e2 != cudaSuccess) {
        (void)cudaGetLastError();
        usable = false;
        why_not_ = std::string("cannot map peer memory: ") + cudaGetErrorString(e1 != cudaSuccess ? e1 : e2);
        if (pa) cudaIpcCloseMemHandle(pa);
        break;
      }
      opened_.push_back(pa);
      opened_.push_back(pp);
      desc_.bufs[r] = pa;
      desc_.sigs[r] = static_cast<uint32_t*>(pp);
    }
  }
  // agree on usability: one failing rank disables the fused path everywhere
  if (world_ > 1) {
    store_->set(key + "/ok/" + std::to_string(rank_), std::vector<uint8_t>{(uint8_t)(usable ? 1 : 0)});
    for (int r = 0; r < world_; ++r) {
      auto v = store_->get(key + "/ok/" + std::to_string(r));
      if (v.empty() || v[0] == 0) {
        if (usable) why_not_ = "a peer could not map this group's memory";
        usable = false;
      }
    }
  }
  if (usable && arena_) {
    int* dev_status = nullptr;
    B200_CUDA_CHECK(cudaHostGetDevicePointer((void**)&dev_status, status_host_, 0));
    desc_.status = dev_status;
  }
  ok_ = usable && arena_ != nullptr;
}

SymmetricMemory::~SymmetricMemory() {
  int cur = -1;
  cudaGetDevice(&cur);
  if (cur != device_) cudaSetDevice(device_);
  cudaDeviceSynchronize();
  for (void* p : opened_) B200_CUDA_WARN(cudaIpcCloseMemHandle(p));
  if (arena_) B200_CUDA_WARN(cudaFree(arena_));
  if (pad_) B200_CUDA_WARN(cudaFree(pad_));
  if (status_host_) B200_CUDA_WARN(cudaFreeHost(status_host_));
  if (cur >= 0 && cur != device_) cudaSetDevice(cur);
}

uint32_t SymmetricMemory::next_epoch(int64_t* half_offset) {
  uint32_t e = epoch_;
  epoch_ += 2;
  if (half_offset) *half_offset = ((e >> 1) & 1) ? (int64_t)half_ : 0;
  return e;
}

int SymmetricMemory::take_status() {
  if (!status_host_) return 0;
  int v = *(volatile int*)status_host_;
  if (v) *(volatile int*)status_host_ = 0;
  return v;
}

at::Tensor SymmetricMemory::local_tensor(int64_t byte_offset, at::IntArrayRef sizes, at::ScalarType dtype) {
  TORCH_CHECK(ok_, "symmetric memory is not available: ", why_not_);
  int64_t n = 1;
  for (auto s : sizes) n *= s;
  TORCH_CHECK(byte_offset >= 0 && (size_t)(byte_offset + n * c10::elementSize(dtype)) <= 2 * half_,
              "symmetric memory: view exceeds the arena");
  return at::from_blob(static_cast<char*>(arena_) + byte_offset, sizes,
                       at::TensorOptions().dtype(dtype).device(make_device(device_)));
}

}  // namespace dist
}  // namespace b200
