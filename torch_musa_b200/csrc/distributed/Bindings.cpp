// Python bindings of the distributed layer: process-group factory, backend-specific controls
// (flight recorder, fused-path switch, test hooks) and symmetric-memory views.
#include "distributed/ProcessGroupBCCL.h"
#include "distributed/SymmetricMemory.h"

#include <pybind11/chrono.h>
#include <torch/csrc/utils/pybind.h>

namespace py = pybind11;

namespace b200 {

void init_distributed_bindings(py::module& m) {
  using dist::ProcessGroupBCCL;
  using dist::SymmetricMemory;

  py::class_<SymmetricMemory, std::shared_ptr<SymmetricMemory>>(m, "_SymmetricMemory")
      .def_property_readonly("ok", &SymmetricMemory::ok)
      .def_property_readonly("why_not", &SymmetricMemory::why_not)
      .def_property_readonly("rank", &SymmetricMemory::rank)
      .def_property_readonly("world", &SymmetricMemory::world)
      .def_property_readonly("half_bytes", &SymmetricMemory::half_bytes)
      .def("take_status", &SymmetricMemory::take_status)
      .def("local_tensor", [](SymmetricMemory& s, int64_t off, std::vector<int64_t> sizes, at::ScalarType dt) {
        return s.local_tensor(off, sizes, dt);
      });

  m.def("_create_process_group", [](c10::intrusive_ptr<c10d::Store> store, int rank, int size,
                                    std::chrono::milliseconds timeout, py::object pg_options) {
    auto opts = c10::make_intrusive<ProcessGroupBCCL::Options>(true);
    opts->timeout = timeout;
    if (!pg_options.is_none()) {
      if (py::hasattr(pg_options, "is_high_priority_stream"))
        opts->is_high_priority_stream = pg_options.attr("is_high_priority_stream").cast<bool>();
      if (py::hasattr(pg_options, "use_fused_collectives"))
        opts->use_fused_collectives = pg_options.attr("use_fused_collectives").cast<bool>();
    }
    c10::intrusive_ptr<c10d::Backend> b = c10::make_intrusive<ProcessGroupBCCL>(std::move(store), rank, size, opts);
    return b;
  });

  auto cast = [](const c10::intrusive_ptr<c10d::Backend>& b) -> ProcessGroupBCCL* {
    auto* p = dynamic_cast<ProcessGroupBCCL*>(b.get());
    TORCH_CHECK(p, "expected a bccl backend object");
    return p;
  };
  m.def("_pg_dump_flight_recorder", [cast](const c10::intrusive_ptr<c10d::Backend>& b) { return cast(b)->dump_flight_recorder(); });
  m.def("_pg_fused_count", [cast](const c10::intrusive_ptr<c10d::Backend>& b) { return cast(b)->fused_collective_count(); });
  m.def("_pg_set_fused", [cast](const c10::intrusive_ptr<c10d::Backend>& b, bool on) { cast(b)->set_fused_collectives(on); });
  m.def("_pg_nccl_version", [cast](const c10::intrusive_ptr<c10d::Backend>& b) { return cast(b)->nccl_version(); });
  m.def("_pg_symmetric_memory", [cast](const c10::intrusive_ptr<c10d::Backend>& b, int device) {
    return cast(b)->symmetric_memory((c10::DeviceIndex)device);
  });
  m.def("_pg_make_test_work", [cast](const c10::intrusive_ptr<c10d::Backend>& b, std::chrono::milliseconds timeout) {
    return cast(b)->make_test_work(timeout);
  });
  m.def("_pg_error", [cast](const c10::intrusive_ptr<c10d::Backend>& b) { return (int)cast(b)->getError(); });
  m.def("_pg_comm_stream", [cast](const c10::intrusive_ptr<c10d::Backend>& b, int device) {
    auto s = cast(b)->comm_stream((c10::DeviceIndex)device).unwrap();
    return py::make_tuple((int64_t)s.id(), (int64_t)s.device_index(), (int64_t)s.device_type());
  });
  m.def("_nccl_version", [] {
    int v = 0;
    ncclGetVersion(&v);
    return v;
  });
}

}  // namespace b200
