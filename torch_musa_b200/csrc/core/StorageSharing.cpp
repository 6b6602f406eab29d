// Sharing device storages between processes (torch.multiprocessing queues and pipes).
//
// A storage that lives in a cudaMalloc segment travels as the cudaIpc handle of the segment plus
// its offset; one that lives in an expandable segment travels as the POSIX file descriptors of
// the physical chunks under it, which the receiver maps into address space of its own.  The
// receiver's DataPtr keeps the mapping open and, when it dies, decrements a reference counter in
// a small shared-memory file; the sender holds the tensor until that counter is back to zero.
//
// Parity: reference torch_musa/csrc/core/StorageSharing.cpp:63-323 (_share_musa_, _new_shared_musa,
// _release_ipc_counter_musa, _edit_device_musa) and MusaIPCTypes.h:11-130 (ref-counter files, limbo).
#include "core/CachingAllocator.h"
#include "core/Device.h"
#include "core/Stream.h"

#include <ATen/ATen.h>
#include <c10/core/TensorImpl.h>
#include <torch/csrc/utils/pybind.h>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <map>
#include <memory>
#include <mutex>

namespace b200 {
namespace {

// ---- reference counters: one 8-byte file under /dev/shm per shared storage
int64_t counter_op(const std::string& path, int64_t delta, bool create) {
  int fd = ::open(path.c_str(), create ? (O_RDWR | O_CREAT | O_EXCL) : O_RDWR, 0600);
  TORCH_CHECK(fd >= 0, "cannot open the IPC reference counter ", path, ": ", std::strerror(errno));
  if (create) TORCH_CHECK(::ftruncate(fd, sizeof(int64_t)) == 0, "cannot size ", path);
  void* m = ::mmap(nullptr, sizeof(int64_t), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  ::close(fd);
  TORCH_CHECK(m != MAP_FAILED, "cannot map ", path);
  auto* w = static_cast<std::atomic<int64_t>*>(m);
  int64_t v = w->fetch_add(delta, std::memory_order_acq_rel) + delta;
  ::munmap(m, sizeof(int64_t));
  return v;
}

// ---- mappings of memory that belongs to another process
struct Mapping {
  int device = 0;
  void* base = nullptr;
  bool is_ipc = true;
  size_t chunk = 0;
  std::vector<uint64_t> handles;
  ~Mapping() {
    if (!base) return;
    if (is_ipc) {
      DeviceSwitch sw(device);
      B200_CUDA_WARN(cudaIpcCloseMemHandle(base));
    } else {
      alloc::get()->unmap_imported(base, chunk, device, handles);
    }
  }
};
std::mutex g_mu;
// One cudaIpc mapping per exporting segment: opening the same handle twice in a process is an error.
std::map<std::string, std::weak_ptr<Mapping>> g_open;

struct Received {
  std::shared_ptr<Mapping> mapping;
  std::string counter;
};
void received_deleter(void* ctx) {
  auto* r = static_cast<Received*>(ctx);
  {
    // the last storage of a segment closes its mapping
    std::lock_guard<std::mutex> g(g_mu);
    r->mapping.reset();
  }
  if (!r->counter.empty()) {
    try {
      counter_op(r->counter, -1, false);
    } catch (...) {
      // the sender is gone and took the file with it
    }
  }
  delete r;
}

py::dict share_storage(const at::Tensor& t) {
  TORCH_CHECK(t.device().type() == kDeviceType, "_share_storage expects a blackwell tensor");
  int device = t.device().index();
  void* p = t.storage().mutable_data();
  TORCH_CHECK(p && alloc::get()->owns(p), "only storages of the caching allocator can be shared between processes");
  {
    // what the sender queued so far must be visible to a receiver that reads on its own streams
    DeviceSwitch sw(device);
    B200_CUDA_CHECK(cudaStreamSynchronize(get_current_stream((c10::DeviceIndex)device).stream()));
  }
  py::dict d;
  d["device"] = device;
  d["nbytes"] = (size_t)t.storage().nbytes();
  d["pid"] = (int64_t)::getpid();
  alloc::CachingAllocator::ShareInfo si;
  if (alloc::get()->share_expandable(p, &si)) {
    d["kind"] = "fd";
    d["fds"] = si.fds;  // the caller owns (and closes) these
    d["chunk_bytes"] = si.chunk_bytes;
    d["offset"] = si.offset;
    return d;
  }
  size_t base_size = 0;
  void* base = alloc::get()->base_allocation(p, &base_size);
  cudaIpcMemHandle_t h;
  {
    DeviceSwitch sw(device);
    B200_CUDA_CHECK(cudaIpcGetMemHandle(&h, base));
  }
  d["kind"] = "ipc";
  d["handle"] = py::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
  d["base_bytes"] = base_size;
  d["offset"] = (size_t)(static_cast<char*>(p) - static_cast<char*>(base));
  return d;
}

at::Tensor wrap(std::shared_ptr<Mapping> m, size_t offset, size_t nbytes, const std::string& counter) {
  auto* r = new Received{std::move(m), counter};
  void* p = static_cast<char*>(r->mapping->base) + offset;
  c10::DataPtr dp(p, r, &received_deleter, make_device(r->mapping->device));
  c10::Storage st(c10::Storage::use_byte_size_t(), nbytes, std::move(dp), /*allocator=*/nullptr, /*resizable=*/false);
  auto out = at::detail::make_tensor<c10::TensorImpl>(std::move(st), c10::DispatchKeySet(c10::DispatchKey::PrivateUse1),
                                                      caffe2::TypeMeta::Make<uint8_t>());
  out.unsafeGetTensorImpl()->set_sizes_contiguous({(int64_t)nbytes});
  return out;
}

at::Tensor open_ipc(int device, const std::string& handle, size_t offset, size_t nbytes, const std::string& counter) {
  TORCH_CHECK(handle.size() == sizeof(cudaIpcMemHandle_t), "bad IPC memory handle size");
  std::shared_ptr<Mapping> m;
  {
    std::lock_guard<std::mutex> g(g_mu);
    auto it = g_open.find(handle);
    if (it != g_open.end()) m = it->second.lock();
    if (!m) {
      cudaIpcMemHandle_t h;
      std::memcpy(&h, handle.data(), sizeof(h));
      DeviceSwitch sw(device);
      void* base = nullptr;
      B200_CUDA_CHECK(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
      m = std::make_shared<Mapping>();
      m->device = device;
      m->base = base;
      m->is_ipc = true;
      g_open[handle] = m;
    }
  }
  return wrap(std::move(m), offset, nbytes, counter);
}

at::Tensor open_fds(int device, const std::vector<int>& fds, size_t chunk, size_t offset, size_t nbytes,
                    const std::string& counter) {
  auto m = std::make_shared<Mapping>();
  m->device = device;
  m->is_ipc = false;
  m->chunk = chunk;
  m->base = alloc::get()->map_imported(fds, chunk, device, &m->handles);
  for (int fd : fds) ::close(fd);  // the mapping holds its own reference to the memory
  return wrap(std::move(m), offset, nbytes, counter);
}

}  // namespace

void init_storage_sharing_bindings(py::module& m) {
  m.def("_share_storage", &share_storage);
  m.def("_open_shared_ipc", &open_ipc, py::arg("device"), py::arg("handle"), py::arg("offset"), py::arg("nbytes"),
        py::arg("counter"));
  m.def("_open_shared_fds", &open_fds, py::arg("device"), py::arg("fds"), py::arg("chunk_bytes"), py::arg("offset"),
        py::arg("nbytes"), py::arg("counter"));
  m.def("_ipc_counter_create", [](const std::string& path, int64_t initial) { return counter_op(path, initial, true); });
  m.def("_ipc_counter_add", [](const std::string& path, int64_t delta) { return counter_op(path, delta, false); });
  m.def("_ipc_counter_unlink", [](const std::string& path) { return ::unlink(path.c_str()) == 0; });
  m.def("_edit_storage_device", [](const at::Tensor& t, int device) {
    // relabels which GPU a storage belongs to (a receiver whose device numbering differs from the sender's)
    t.storage().mutable_data_ptr().unsafe_set_device(make_device(device));
  });
  m.def("_open_mapping_count", [] {
    std::lock_guard<std::mutex> g(g_mu);
    int n = 0;
    for (auto& kv : g_open) n += kv.second.expired() ? 0 : 1;
    return n;
  });
}

}  // namespace b200
