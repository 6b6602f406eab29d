// CPython bindings: torch_musa_b200._C.  Thin wrappers over the runtime layer;
// every policy decision lives in the C++ classes or in the Python frontend.
// Parity: reference torch_musa/csrc/core/Module.cpp:950-1058,1418-1465, Stream.cpp,
// Event.cpp, Graph.cpp:10-72.
#include "aten/CudaAlias.h"
#include "aten/Ops.h"
#include "core/Backend.h"
#include "core/CachingAllocator.h"
#include "core/Device.h"
#include "core/DeviceAssert.h"
#include "core/Generator.h"
#include "core/Graph.h"
#include "core/HostAllocator.h"
#include "core/Stream.h"

#include <ATen/cuda/CUDAGeneratorImpl.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <torch/csrc/Generator.h>
#include <torch/csrc/utils/pybind.h>
#include <torch/csrc/utils/python_numbers.h>

#include <dlfcn.h>
#include <pthread.h>

namespace py = pybind11;
using namespace b200;

namespace b200 {
void init_distributed_bindings(py::module& m);
void init_storage_sharing_bindings(py::module& m);
void init_compile_bindings(py::module& m);
}

namespace {

bool g_in_bad_fork = false;
bool g_fork_handler_registered = false;

void forked_child() { g_in_bad_fork = true; }

void poison_fork() {
  if (g_fork_handler_registered) return;
  pthread_atfork(nullptr, nullptr, forked_child);
  g_fork_handler_registered = true;
}

py::dict stat_to_dict(const alloc::Stat& s) {
  py::dict d;
  d["current"] = s.current;
  d["peak"] = s.peak;
  d["allocated"] = s.allocated;
  d["freed"] = s.freed;
  return d;
}

py::dict stat_array(const alloc::Stat* arr) {
  static const char* names[] = {"all", "small_pool", "large_pool"};
  py::dict d;
  for (int i = 0; i < alloc::kNumStatTypes; ++i) d[names[i]] = stat_to_dict(arr[i]);
  return d;
}

py::dict memory_stats(int device) {
  auto s = alloc::get()->stats(device);
  py::dict d;
  d["num_alloc_retries"] = s.num_alloc_retries;
  d["num_ooms"] = s.num_ooms;
  d["max_split_size"] = s.max_split_size;
  d["num_sync_all_streams"] = s.num_sync_all_streams;
  d["num_device_alloc"] = s.num_device_alloc;
  d["num_device_free"] = s.num_device_free;
  d["allocation"] = stat_array(s.allocation);
  d["segment"] = stat_array(s.segment);
  d["active"] = stat_array(s.active);
  d["inactive_split"] = stat_array(s.inactive_split);
  d["allocated_bytes"] = stat_array(s.allocated_bytes);
  d["reserved_bytes"] = stat_array(s.reserved_bytes);
  d["active_bytes"] = stat_array(s.active_bytes);
  d["inactive_split_bytes"] = stat_array(s.inactive_split_bytes);
  d["requested_bytes"] = stat_array(s.requested_bytes);
  d["oversize_allocations"] = stat_to_dict(s.oversize_allocations);
  d["oversize_segments"] = stat_to_dict(s.oversize_segments);
  return d;
}

py::list snapshot(int device) {
  py::list out;
  for (auto& seg : alloc::get()->snapshot(device)) {
    py::dict d;
    d["device"] = seg.device;
    d["address"] = seg.address;
    d["total_size"] = seg.total_size;
    d["allocated_size"] = seg.allocated_size;
    d["active_size"] = seg.active_size;
    d["requested_size"] = seg.requested_size;
    d["stream"] = (uintptr_t)seg.stream;
    d["segment_type"] = seg.is_large ? "large" : "small";
    d["segment_pool_id"] = py::make_tuple(seg.pool_id_first, seg.pool_id_second);
    d["is_expandable"] = seg.is_expandable;
    py::list blocks;
    for (auto& b : seg.blocks) {
      py::dict bd;
      bd["address"] = b.address;
      bd["size"] = b.size;
      bd["requested_size"] = b.requested;
      bd["state"] = b.allocated ? "active_allocated" : (b.active ? "active_pending_free" : "inactive");
      blocks.append(bd);
    }
    d["blocks"] = blocks;
    out.append(d);
  }
  return out;
}

py::list trace(int device) {
  static const char* names[] = {"alloc", "free_requested", "free_completed", "segment_alloc", "segment_free", "oom",
                                "snapshot"};
  py::list out;
  for (auto& t : alloc::get()->trace(device)) {
    py::dict d;
    d["action"] = names[(int)t.action];
    d["addr"] = t.addr;
    d["size"] = t.size;
    d["stream"] = (uintptr_t)t.stream;
    d["device"] = t.device;
    d["time_us"] = t.time_ns / 1000;
    if (!t.stack.empty()) d["frames"] = t.stack;
    out.append(d);
  }
  return out;
}

py::dict props_dict(int d) {
  const cudaDeviceProp& p = device_properties((c10::DeviceIndex)d);
  py::dict r;
  r["name"] = std::string(p.name);
  r["major"] = p.major;
  r["minor"] = p.minor;
  r["total_memory"] = (size_t)p.totalGlobalMem;
  r["multi_processor_count"] = p.multiProcessorCount;
  r["warp_size"] = p.warpSize;
  r["max_threads_per_multi_processor"] = p.maxThreadsPerMultiProcessor;
  r["max_threads_per_block"] = p.maxThreadsPerBlock;
  r["regs_per_multiprocessor"] = p.regsPerMultiprocessor;
  r["shared_memory_per_block"] = (size_t)p.sharedMemPerBlock;
  r["shared_memory_per_block_optin"] = (size_t)p.sharedMemPerBlockOptin;
  r["shared_memory_per_multiprocessor"] = (size_t)p.sharedMemPerMultiprocessor;
  r["l2_cache_size"] = p.l2CacheSize;
  r["is_integrated"] = p.integrated != 0;
  r["is_multi_gpu_board"] = p.isMultiGpuBoard != 0;
  r["pci_bus_id"] = p.pciBusID;
  r["pci_device_id"] = p.pciDeviceID;
  r["pci_domain_id"] = p.pciDomainID;
  char uuid[33];
  for (int i = 0; i < 16; ++i) snprintf(uuid + 2 * i, 3, "%02x", (unsigned char)p.uuid.bytes[i]);
  r["uuid"] = std::string(uuid);
  return r;
}

// pluggable allocator: function pointers from a user .so
using PlugAlloc = void* (*)(size_t, int, cudaStream_t);
using PlugFree = void (*)(void*, size_t, int, cudaStream_t);
PlugAlloc g_plug_alloc = nullptr;
PlugFree g_plug_free = nullptr;
int plug_alloc_tramp(void** p, size_t n, int dev, cudaStream_t s) {
  *p = g_plug_alloc(n, dev, s);
  return *p ? 0 : (int)cudaErrorMemoryAllocation;
}
int plug_free_tramp(void* p, size_t n, int dev, cudaStream_t s) {
  g_plug_free(p, n, dev, s);
  return 0;
}

std::vector<py::object> g_oom_callbacks;

}  // namespace

PYBIND11_MODULE(_C, m) {
  m.doc() = "torch_musa_b200 native runtime";

  // ------------------------------------------------------------ init / device
  m.def("_register_hooks", [] { register_hooks(); });
  m.def("_init", [] {
    TORCH_CHECK(!g_in_bad_fork, "Cannot re-initialize blackwell in forked subprocess. To use blackwell with "
                                "multiprocessing, you must use the 'spawn' start method");
    poison_fork();
    lazy_init();
  });
  m.def("_is_initialized", [] { return is_initialized(); });
  m.def("_device_type_enum", [] { return (int64_t)kDeviceType; });
  m.def("_is_in_bad_fork", [] { return g_in_bad_fork; });
  m.def("_device_count", [] { return (int)device_count(); });
  m.def("_current_device", [] { return (int)current_device(); });
  m.def("_set_device", [](int d) { set_device((c10::DeviceIndex)d); });
  m.def("_exchange_device", [](int d) { return d < 0 ? -1 : (int)exchange_device((c10::DeviceIndex)d); });
  m.def("_maybe_exchange_device", [](int d) { return d < 0 ? -1 : (int)maybe_exchange_device((c10::DeviceIndex)d); });
  m.def("_synchronize", [] {
    py::gil_scoped_release nogil;
    device_synchronize();
  });
  m.def("_device_properties", &props_dict);
  m.def("_can_access_peer", [](int a, int b) { return can_access_peer((c10::DeviceIndex)a, (c10::DeviceIndex)b); });
  m.def("_enable_peer_access", [](int a, int b) { return enable_peer_access((c10::DeviceIndex)a, (c10::DeviceIndex)b); });
  m.def("_has_primary_context", [](int d) { return has_primary_context((c10::DeviceIndex)d); });
  m.def("_set_sync_debug_mode", &set_sync_debug_mode);
  m.def("_get_sync_debug_mode", &sync_debug_mode);
  m.def("_launch_blocking", &launch_blocking);
  m.def("_sleep", [](int64_t cycles) { B200_KERNEL_CALL(b200_sleep(cycles, get_current_stream().stream())); });
  m.def("_kernels_arch", [] { return std::string(b200_kernels_arch()); });
  m.def("_kernel_launch_count", [] { return b200_launch_count(); });
  m.def("_reset_kernel_launch_count", [] { b200_reset_launch_count(); });
  m.def("_gemm_available", [] { return b200_gemm_available() != 0; });
  m.def("_gemm_status", [](bool clear) { return b200_gemm_status(clear ? 1 : 0); }, py::arg("clear") = false);
  m.def("_set_pointwise_conv_gemm", [](bool on) { ops::set_pointwise_conv_gemm(on); });
  m.def("_pointwise_conv_hits", [] { return ops::pointwise_conv_hits(); });
  m.def("_set_implicit_conv_gemm", [](bool on) { ops::set_implicit_conv_gemm(on); });
  m.def("_implicit_conv_hits", [] { return ops::implicit_conv_hits(); });
  m.def("_conv_status", [](bool clear) { return b200_conv_status(clear ? 1 : 0); });
  m.def("_gemm_force_config", [](int c) { return b200_gemm_force_config(c); });
  m.def("_set_tensor_core_gemm", [](bool on) { ops::set_tensor_core_gemm(on); });
  m.def("_set_fused_sdp", [](bool on) { ops::set_fused_sdp(on); });
  m.def("_set_sdp_impl", [](int impl) { ops::set_sdp_impl(impl); });
  m.def("_sdp_impl", [] { return ops::sdp_impl(); });
  m.def("_take_device_assert", [](int dev) { return take_device_assert((c10::DeviceIndex)dev); });
  m.def("_native_sdp_forward_calls", [] { return ops::native_sdp_forward_calls(); });
  m.def("_native_sdp_backward_calls", [] { return ops::native_sdp_backward_calls(); });
  m.def("_fused_sdp_enabled", [] { return ops::fused_sdp_enabled(); });
  m.def("_tensor_core_gemm_enabled", [] { return ops::tensor_core_gemm_enabled(); });
  m.def("_runtime_version", [] {
    int v = 0;
    cudaRuntimeGetVersion(&v);
    return v;
  });
  m.def("_driver_version", [] {
    int v = 0;
    if (cudaDriverGetVersion(&v) != cudaSuccess) (void)cudaGetLastError();
    return v;
  });

  // ------------------------------------------------------------ streams
  m.def("_current_stream", [](int d) {
    auto s = get_current_stream((c10::DeviceIndex)d).unwrap();
    return py::make_tuple((int64_t)s.id(), (int64_t)s.device_index(), (int64_t)s.device_type());
  });
  m.def("_default_stream", [](int d) {
    auto s = get_default_stream((c10::DeviceIndex)d).unwrap();
    return py::make_tuple((int64_t)s.id(), (int64_t)s.device_index(), (int64_t)s.device_type());
  });
  m.def("_set_stream", [](int64_t id, int64_t dev, int64_t type) {
    auto s = c10::Stream::unpack3(id, (c10::DeviceIndex)dev, (c10::DeviceType)type);
    Stream bs(s);
    if (current_device() != bs.device_index()) set_device(bs.device_index());
    set_current_stream(bs);
  });
  m.def("_stream_from_pool", [](int priority, int d) {
    auto s = get_stream_from_pool(priority, (c10::DeviceIndex)d).unwrap();
    return py::make_tuple((int64_t)s.id(), (int64_t)s.device_index(), (int64_t)s.device_type());
  });
  m.def("_stream_from_external", [](uintptr_t ptr, int d) {
    auto s = get_stream_from_external(reinterpret_cast<cudaStream_t>(ptr), (c10::DeviceIndex)d).unwrap();
    return py::make_tuple((int64_t)s.id(), (int64_t)s.device_index(), (int64_t)s.device_type());
  });
  m.def("_stream_handle", [](int64_t id, int64_t dev) {
    auto s = c10::Stream::unpack3(id, (c10::DeviceIndex)dev, kDeviceType);
    return (uintptr_t)stream_from_c10(s);
  });
  m.def("_stream_priority", [](int64_t id, int64_t dev) {
    return Stream(c10::Stream::unpack3(id, (c10::DeviceIndex)dev, kDeviceType)).priority();
  });
  m.def("_stream_priority_range", [] {
    int l, g;
    priority_range(&l, &g);
    return py::make_tuple(l, g);
  });
  m.def("_stream_synchronize", [](int64_t id, int64_t dev) {
    py::gil_scoped_release nogil;
    Stream(c10::Stream::unpack3(id, (c10::DeviceIndex)dev, kDeviceType)).synchronize();
  });
  m.def("_stream_is_capturing", [](int64_t id, int64_t dev) {
    return Graph::is_capturing(stream_from_c10(c10::Stream::unpack3(id, (c10::DeviceIndex)dev, kDeviceType)));
  });

  m.def("_event_elapsed_time", [](uintptr_t a, uintptr_t b) {
    TORCH_CHECK(a && b, "Both events must be recorded before calculating elapsed time.");
    float ms = 0.f;
    B200_CUDA_CHECK(cudaEventElapsedTime(&ms, reinterpret_cast<cudaEvent_t>(a), reinterpret_cast<cudaEvent_t>(b)));
    return ms;
  });

  // IPC-capable event (the generic torch.Event covers everything else)
  py::class_<Event>(m, "_IpcEvent")
      .def(py::init([](bool interprocess, bool timing) {
        unsigned f = timing ? cudaEventDefault : cudaEventDisableTiming;
        if (interprocess) f |= cudaEventInterprocess | cudaEventDisableTiming;
        return new Event(f);
      }), py::arg("interprocess") = true, py::arg("enable_timing") = false)
      .def_static("from_ipc_handle", [](int device, py::bytes h) {
        std::string s = h;
        TORCH_CHECK(s.size() == sizeof(cudaIpcEventHandle_t), "bad IPC event handle size");
        cudaIpcEventHandle_t hh;
        memcpy(&hh, s.data(), sizeof(hh));
        return new Event(Event::from_ipc_handle((c10::DeviceIndex)device, &hh));
      })
      .def("ipc_handle", [](Event& e) {
        cudaIpcEventHandle_t h;
        e.ipc_handle(&h);
        return py::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
      })
      .def("record", [](Event& e, int64_t id, int64_t dev) {
        e.record(Stream(c10::Stream::unpack3(id, (c10::DeviceIndex)dev, kDeviceType)));
      })
      .def("wait", [](Event& e, int64_t id, int64_t dev) {
        e.block(Stream(c10::Stream::unpack3(id, (c10::DeviceIndex)dev, kDeviceType)));
      })
      .def("query", &Event::query)
      .def("synchronize", [](Event& e) {
        py::gil_scoped_release nogil;
        e.synchronize();
      })
      .def("elapsed_time", [](Event& a, Event& b) { return a.elapsed_ms(b); })
      .def_property_readonly("device_index", [](Event& e) { return (int)e.device_index(); });

  // ------------------------------------------------------------ memory
  m.def("_empty_cache", [](int device) {
    alloc::get()->empty_cache(device);
    if (device_count() > 0) c10::cuda::CUDACachingAllocator::emptyCache();
  }, py::arg("device") = -1);
  m.def("_memory_stats", &memory_stats);
  m.def("_reset_accumulated_memory_stats", [](int d) { alloc::get()->reset_accumulated_stats(d); });
  m.def("_reset_peak_memory_stats", [](int d) { alloc::get()->reset_peak_stats(d); });
  m.def("_mem_get_info", [](int d) {
    size_t f = 0, t = 0;
    alloc::get()->mem_info(d, &f, &t);
    return py::make_tuple(f, t);
  });
  m.def("_set_memory_fraction", [](double f, int d) { alloc::get()->set_memory_fraction(f, d); });
  m.def("_get_memory_fraction", [](int d) { return alloc::get()->get_memory_fraction(d); });
  m.def("_snapshot", &snapshot, py::arg("device") = -1);
  m.def("_trace", &trace);
  m.def("_record_memory_history", [](bool on, size_t max_entries, bool stacks) {
    alloc::get()->record_history(on, max_entries, stacks);
  }, py::arg("enabled"), py::arg("max_entries"), py::arg("stacks") = false);
  m.def("_allocator_backend", [] { return alloc::backend_name(); });
  m.def("_set_allocator_settings", [](const std::string& s) { alloc::set_config_string(s); });
  m.def("_allocator_config", [] {
    const auto& c = alloc::config();
    py::dict d;
    d["max_split_size"] = c.max_split_size == SIZE_MAX ? py::object(py::none()) : py::object(py::int_(c.max_split_size));
    d["garbage_collection_threshold"] = c.gc_threshold;
    d["roundup_power2_divisions"] = c.roundup_power2_divisions;
    d["large_segment_bytes"] = c.large_segment_bytes;
    d["expandable_segments"] = c.expandable_segments;
    d["canary"] = c.canary;
    d["backend"] = c.backend;
    d["cpu_unified"] = c.cpu_unified;
    d["no_caching"] = c.no_caching;
    d["pinned_use_host_register"] = c.pinned_use_host_register;
    d["pinned_num_register_threads"] = c.pinned_num_register_threads;
    return d;
  });
  m.def("_parse_allocator_config", [](const std::string& s) {
    auto c = alloc::parse_config(s);
    py::dict d;
    d["max_split_size"] = c.max_split_size == SIZE_MAX ? py::object(py::none()) : py::object(py::int_(c.max_split_size));
    d["garbage_collection_threshold"] = c.gc_threshold;
    d["roundup_power2_divisions"] = c.roundup_power2_divisions;
    d["large_segment_bytes"] = c.large_segment_bytes;
    d["expandable_segments"] = c.expandable_segments;
    d["canary"] = c.canary;
    d["backend"] = c.backend;
    d["cpu_unified"] = c.cpu_unified;
    d["pinned_use_host_register"] = c.pinned_use_host_register;
    d["pinned_num_register_threads"] = c.pinned_num_register_threads;
    d["pinned_use_background_threads"] = c.pinned_use_background_threads;
    d["release_lock_on_malloc"] = c.release_lock_on_malloc;
    return d;
  });
  m.def("_raw_alloc", [](size_t n, int d, uintptr_t stream) {
    lazy_init();
    return (uintptr_t)alloc::get()->raw_alloc(n, d, reinterpret_cast<cudaStream_t>(stream));
  });
  m.def("_raw_delete", [](uintptr_t p) { alloc::get()->raw_delete(reinterpret_cast<void*>(p)); });
  m.def("_host_stats", [] {
    auto s = host::stats();
    py::dict d;
    d["allocations"] = s.allocations; d["frees"] = s.frees; d["cached_blocks"] = s.cached_blocks;
    d["cached_bytes"] = s.cached_bytes; d["active_blocks"] = s.active_blocks; d["active_bytes"] = s.active_bytes;
    d["device_allocs"] = s.device_allocs; d["reuse_hits"] = s.reuse_hits; d["events_pending"] = s.events_pending;
    return d;
  });
  m.def("_host_empty_cache", [] { host::empty_cache(); });
  m.def("_set_unified_cpu_allocator", [](bool on) { host::set_unified_cpu_allocator(on); });
  m.def("_unified_cpu_allocator_enabled", [] { return host::unified_cpu_allocator_enabled(); });
  m.def("_is_managed_ptr", [](uintptr_t p) { return host::is_managed_ptr(reinterpret_cast<const void*>(p)); });
  m.def("_managed_storage_to_device", [](const at::Storage& s, int idx) {
    TORCH_CHECK(s.device().is_cpu() && host::is_managed_ptr(s.data()), "storage is not in managed host memory");
    return bridge::relabel_storage(s, make_device((c10::DeviceIndex)idx));
  });
  m.def("_allocator_canary_violations", [] { return alloc::get()->canary_violations(); });
  m.def("_allocator_last_canary_report", [] { return alloc::get()->last_canary_report(); });
  m.def("_event_cache_stats", [] { return event_cache_stats(); });
  m.def("_multi_stream_guard_probe", [](std::vector<std::tuple<int64_t, int64_t>> ids) {
    // sets the given streams current on their devices inside a MultiStreamGuard and reports what was current
    // inside and after the guard (used by the tests of the guard classes)
    std::vector<Stream> streams;
    for (auto& t : ids) streams.emplace_back(c10::Stream::unpack3(std::get<0>(t), (c10::DeviceIndex)std::get<1>(t), kDeviceType));
    std::vector<int64_t> inside, after;
    {
      MultiStreamGuard g(streams);
      OptionalStreamGuard og;
      if (!streams.empty()) og.reset_stream(streams.front());
      for (auto& s : streams) inside.push_back(get_current_stream(s.device_index()).id());
    }
    for (auto& s : streams) after.push_back(get_current_stream(s.device_index()).id());
    return py::make_tuple(inside, after);
  });
  m.def("_host_register", [](uintptr_t p, size_t n) {
    B200_CUDA_CHECK(cudaHostRegister(reinterpret_cast<void*>(p), n, cudaHostRegisterDefault));
  });
  m.def("_host_unregister", [](uintptr_t p) { B200_CUDA_CHECK(cudaHostUnregister(reinterpret_cast<void*>(p))); });
  m.def("_install_pluggable_allocator", [](const std::string& path, const std::string& alloc_name,
                                           const std::string& free_name) {
    void* h = dlopen(path.c_str(), RTLD_LAZY | RTLD_LOCAL);
    TORCH_CHECK(h, "cannot load allocator library ", path, ": ", dlerror());
    g_plug_alloc = (PlugAlloc)dlsym(h, alloc_name.c_str());
    g_plug_free = (PlugFree)dlsym(h, free_name.c_str());
    TORCH_CHECK(g_plug_alloc && g_plug_free, "symbols ", alloc_name, "/", free_name, " not found in ", path);
    alloc::install_pluggable(&plug_alloc_tramp, &plug_free_tramp);
  });
  m.def("_attach_oom_observer", [](py::object cb) {
    g_oom_callbacks.push_back(cb);
    size_t idx = g_oom_callbacks.size() - 1;
    alloc::get()->attach_oom_observer([idx](int device, size_t req, size_t total, size_t free_b) {
      py::gil_scoped_acquire gil;
      try {
        g_oom_callbacks[idx](device, req, total, free_b);
      } catch (py::error_already_set& e) {
        e.discard_as_unraisable("blackwell OOM observer");
      }
    });
  });
  m.def("_new_mempool_id", [](bool user) {
    auto id = alloc::CachingAllocator::new_pool_id(user);
    return py::make_tuple(id.first, id.second);
  });
  m.def("_begin_allocate_to_pool", [](int device, std::pair<uint64_t, uint64_t> id) {
    // route allocations of the *calling thread's current stream* to the pool
    cudaStream_t cs = get_current_stream((c10::DeviceIndex)device).stream();
    alloc::get()->create_or_incref_pool(device, id);
    alloc::get()->begin_allocate_to_pool(device, id, [cs](cudaStream_t s) { return s == cs; });
  });
  m.def("_end_allocate_to_pool", [](int device, std::pair<uint64_t, uint64_t> id) {
    alloc::get()->end_allocate_to_pool(device, id);
  });
  m.def("_release_pool", [](int device, std::pair<uint64_t, uint64_t> id) { alloc::get()->release_pool(device, id); });
  m.def("_pool_use_count", [](int device, std::pair<uint64_t, uint64_t> id) {
    return alloc::get()->pool_use_count(device, id);
  });

  // Private-pool checkpoints.  `stale` tensors lose their claim on memory the restore took back (their deleter
  // becomes a no-op); `adopt` tensors, whose data pointers the restore re-created, get a deleter that frees them.
  py::class_<alloc::PoolCheckpoint>(m, "_PoolCheckpoint")
      .def_property_readonly("device", [](const alloc::PoolCheckpoint& c) { return c.device; })
      .def_property_readonly("pool", [](const alloc::PoolCheckpoint& c) { return c.pool; })
      .def_property_readonly("live_pointers", [](const alloc::PoolCheckpoint& c) {
        std::vector<uintptr_t> v;
        for (auto& s : c.segments)
          for (auto& b : s.blocks)
            if (b.allocated) v.push_back(b.address);
        return v;
      });
  m.def("_checkpoint_pool", [](int device, std::pair<uint64_t, uint64_t> id) {
    return alloc::get()->checkpoint_pool(device, id);
  });
  m.def("_restore_pool", [](int device, const alloc::PoolCheckpoint& state, std::vector<at::Tensor> stale) {
    auto* a = alloc::get();
    auto res = a->restore_pool(device, state);
    c10::DeleterFnPtr real = a->raw_deleter(), noop = alloc::CachingAllocator::noop_deleter();
    for (auto& t : stale) t.storage().mutable_data_ptr().compare_exchange_deleter(real, noop);
    std::vector<uintptr_t> fr, al;
    for (void* p : res.freed) fr.push_back((uintptr_t)p);
    for (void* p : res.allocated) al.push_back((uintptr_t)p);
    return py::make_tuple(fr, al);
  }, py::arg("device"), py::arg("state"), py::arg("stale") = std::vector<at::Tensor>());
  m.def("_adopt_allocation", [](int device, uintptr_t ptr, size_t nbytes) {
    // A byte tensor that owns a live allocation nobody owns yet (one that a pool restore re-created).
    c10::DataPtr dp = alloc::get()->adopt(reinterpret_cast<void*>(ptr), device);
    c10::Storage st(c10::Storage::use_byte_size_t(), nbytes, std::move(dp), nullptr, false);
    auto out = at::detail::make_tensor<c10::TensorImpl>(std::move(st), c10::DispatchKeySet(c10::DispatchKey::PrivateUse1),
                                                        caffe2::TypeMeta::Make<uint8_t>());
    out.unsafeGetTensorImpl()->set_sizes_contiguous({(int64_t)nbytes});
    return out;
  });

  // A caching allocator over plain host memory (events complete immediately): lets the cache logic
  // (rounding, pools, split/merge, stream affinity, private pools, fraction, OOM retry) be unit-tested
  // on machines without a GPU.
  struct HostCacheHarness {
    std::unique_ptr<alloc::CachingAllocator> a;
  };
  py::class_<HostCacheHarness>(m, "_HostCacheHarness")
      .def(py::init([] {
        auto* h = new HostCacheHarness();
        h->a = std::make_unique<alloc::CachingAllocator>(alloc::host_backend(), 1);
        return h;
      }))
      .def("alloc", [](HostCacheHarness& h, size_t n, uintptr_t stream) {
        return (uintptr_t)h.a->raw_alloc(n, 0, reinterpret_cast<cudaStream_t>(stream));
      }, py::arg("nbytes"), py::arg("stream") = 0)
      .def("free", [](HostCacheHarness& h, uintptr_t p) { h.a->raw_delete(reinterpret_cast<void*>(p)); })
      .def("record_stream", [](HostCacheHarness& h, uintptr_t p, uintptr_t s) {
        h.a->record_stream_ptr(reinterpret_cast<void*>(p), 0, reinterpret_cast<cudaStream_t>(s));
      })
      .def("empty_cache", [](HostCacheHarness& h) { h.a->empty_cache(0); })
      .def("set_memory_fraction", [](HostCacheHarness& h, double f) { h.a->set_memory_fraction(f, 0); })
      .def("stats", [](HostCacheHarness& h) {
        auto s = h.a->stats(0);
        py::dict d;
        d["allocated_bytes"] = stat_array(s.allocated_bytes);
        d["reserved_bytes"] = stat_array(s.reserved_bytes);
        d["active_bytes"] = stat_array(s.active_bytes);
        d["inactive_split_bytes"] = stat_array(s.inactive_split_bytes);
        d["allocation"] = stat_array(s.allocation);
        d["segment"] = stat_array(s.segment);
        d["num_alloc_retries"] = s.num_alloc_retries;
        d["num_ooms"] = s.num_ooms;
        d["num_device_alloc"] = s.num_device_alloc;
        d["num_device_free"] = s.num_device_free;
        return d;
      })
      .def("snapshot", [](HostCacheHarness& h) {
        py::list out;
        for (auto& seg : h.a->snapshot(0)) {
          py::dict d;
          d["address"] = seg.address;
          d["total_size"] = seg.total_size;
          d["allocated_size"] = seg.allocated_size;
          d["is_large"] = seg.is_large;
          d["pool_id"] = py::make_tuple(seg.pool_id_first, seg.pool_id_second);
          d["is_expandable"] = seg.is_expandable;
          py::list blocks;
          for (auto& b : seg.blocks) blocks.append(py::make_tuple(b.size, b.allocated));
          d["blocks"] = blocks;
          out.append(d);
        }
        return out;
      })
      .def("begin_pool", [](HostCacheHarness& h, std::pair<uint64_t, uint64_t> id, uintptr_t stream) {
        cudaStream_t cs = reinterpret_cast<cudaStream_t>(stream);
        h.a->create_or_incref_pool(0, id);
        h.a->begin_allocate_to_pool(0, id, [cs](cudaStream_t s) { return s == cs; });
      })
      .def("end_pool", [](HostCacheHarness& h, std::pair<uint64_t, uint64_t> id) { h.a->end_allocate_to_pool(0, id); })
      .def("release_pool", [](HostCacheHarness& h, std::pair<uint64_t, uint64_t> id) { h.a->release_pool(0, id); })
      .def("checkpoint", [](HostCacheHarness& h, std::pair<uint64_t, uint64_t> id) { return h.a->checkpoint_pool(0, id); })
      .def("restore", [](HostCacheHarness& h, const alloc::PoolCheckpoint& c) {
        auto res = h.a->restore_pool(0, c);
        std::vector<uintptr_t> fr, al;
        for (void* p : res.freed) fr.push_back((uintptr_t)p);
        for (void* p : res.allocated) al.push_back((uintptr_t)p);
        return py::make_tuple(fr, al);
      })
      .def("write_read", [](HostCacheHarness&, uintptr_t p, size_t n, int value) {
        // touches host-backend memory: proves a mapped range is really usable
        std::memset(reinterpret_cast<void*>(p), value, n);
        return (int)reinterpret_cast<unsigned char*>(p)[n - 1];
      })
      .def("canary_violations", [](HostCacheHarness& h) { return h.a->canary_violations(); })
      .def("last_canary_report", [](HostCacheHarness& h) { return h.a->last_canary_report(); })
      .def("record_history", [](HostCacheHarness& h, bool on, size_t n) { h.a->record_history(on, n); })
      .def("trace", [](HostCacheHarness& h) {
        py::list out;
        for (auto& t : h.a->trace(0)) out.append(py::make_tuple((int)t.action, t.addr, t.size));
        return out;
      });

  // ------------------------------------------------------------ RNG
  m.def("_default_generator", [](int d) {
    lazy_init();
    return py::reinterpret_steal<py::object>(THPGenerator_Wrap(default_generator((c10::DeviceIndex)d)));
  });
  m.def("_seed_cuda_twin", [](int d, uint64_t seed) {
    // long-tail random ops draw from torch's CUDA generator of the same ordinal
    auto g = at::cuda::detail::getDefaultCUDAGenerator((c10::DeviceIndex)d);
    std::lock_guard<std::mutex> lock(g.mutex());
    g.set_current_seed(seed);
  });

  // ------------------------------------------------------------ fallback bookkeeping
  m.def("_fallback_counts", [] { return bridge::fallback_counts(); });
  m.def("_reset_fallback_counts", [] { bridge::reset_fallback_counts(); });
  m.def("_set_fallback_logging", [](int lvl) { bridge::set_fallback_logging(lvl); });

  // ------------------------------------------------------------ graphs
  py::class_<Graph>(m, "_Graph")
      .def(py::init<>())
      .def("capture_begin", [](Graph& g, std::optional<std::pair<uint64_t, uint64_t>> pool, const std::string& mode) {
        cudaStreamCaptureMode cm = cudaStreamCaptureModeGlobal;
        if (mode == "thread_local") cm = cudaStreamCaptureModeThreadLocal;
        else if (mode == "relaxed") cm = cudaStreamCaptureModeRelaxed;
        else TORCH_CHECK(mode == "global", "Unknown capture error mode. Expected `global`, `thread_local`, or `relaxed`, got ", mode);
        g.capture_begin(pool.value_or(std::pair<uint64_t, uint64_t>{0, 0}), cm);
      }, py::arg("pool") = py::none(), py::arg("capture_error_mode") = "global")
      .def("capture_end", [](Graph& g) {
        py::gil_scoped_release nogil;
        g.capture_end();
      })
      .def("replay", [](Graph& g) {
        py::gil_scoped_release nogil;
        g.replay();
      })
      .def("reset", &Graph::reset)
      .def("pool", [](Graph& g) {
        auto p = g.pool();
        return py::make_tuple(p.first, p.second);
      })
      .def("enable_debug_mode", &Graph::enable_debug_mode)
      .def("debug_dump", &Graph::debug_dump)
      .def("reinstantiate_graph", &Graph::reinstantiate);
  m.def("_graph_pool_handle", [] {
    auto p = Graph::new_pool_handle();
    return py::make_tuple(p.first, p.second);
  });

  b200::init_distributed_bindings(m);
  b200::init_storage_sharing_bindings(m);
  b200::init_compile_bindings(m);
}
