// Python bindings of the distributed layer (process group backend, symmetric memory).
#include <torch/csrc/utils/pybind.h>

namespace b200 {
void init_distributed_bindings(pybind11::module& m) { (void)m; }
}  // namespace b200
