// A flat, Python-free executor for traced graphs: the compile stack lowers an FX graph to a list
// of instructions (boxed dispatcher calls, generated fused pointwise kernels, tuple indexing) over
// numbered value slots, with the slot lifetimes planned ahead, and this class runs it without
// touching the interpreter.  It is the run-time half of torch.compile(backend="blackwell") and of
// packages written by export.aot_compile.
//
// Parity: reference torch_musa/csrc/inductor/aoti_runner/model_container_runner_musa.cpp:6-49 (a C++
// runner that executes a compiled model on a device stream) and _inductor wrapper code generation.
#include "compile/Jit.h"
#include "core/Stream.h"

#include <ATen/ATen.h>
#include <ATen/ScalarOps.h>
#include <ATen/core/dispatch/Dispatcher.h>
#include <torch/csrc/jit/python/pybind_utils.h>
#include <torch/csrc/utils/pybind.h>

namespace b200 {
namespace {

struct Arg {
  enum Kind { CONST, SLOT, SLOT_LIST } kind = CONST;
  c10::IValue value;            // CONST
  int slot = -1;                // SLOT
  std::vector<int> slots;       // SLOT_LIST: -1 entries are None (optional tensor lists)
  bool optional_list = false;
};

struct Instr {
  enum Kind { OP, FUSED, GETITEM } kind = OP;
  // OP
  std::optional<c10::OperatorHandle> op;
  std::vector<Arg> args;
  // FUSED
  std::shared_ptr<jit::Kernel> kernel;
  std::vector<int> in_slots;
  std::vector<int64_t> out_shape;
  std::vector<c10::ScalarType> out_dtypes;
  int vec = 1;  // elements per thread of the contiguous fast path (0 = generic indexing only)
  // GETITEM
  int src = -1, index = 0;
  // common
  std::vector<int> out_slots;   // OP: one slot (a tuple if the operator returns several values)
  std::vector<int> free_after;  // slots dead once this instruction has run
  std::string name;
};

class GraphRunner {
 public:
  int n_slots = 0;
  std::vector<int> input_slots, output_slots;  // output slot -1 = None
  std::vector<Instr> prog;
  int64_t runs = 0, fused_launches = 0, op_calls = 0;

  int add_op(const std::string& qualified, const std::string& overload, py::list pyargs, int out_slot,
             std::vector<int> free_after, const std::string& name) {
    Instr in;
    in.kind = Instr::OP;
    in.name = name;
    in.op = c10::Dispatcher::singleton().findSchemaOrThrow(qualified.c_str(), overload.c_str());
    const auto& schema = in.op->schema();
    TORCH_CHECK(pyargs.size() == schema.arguments().size(), name, ": expected ", schema.arguments().size(),
                " normalised arguments, got ", pyargs.size());
    for (size_t i = 0; i < pyargs.size(); ++i) {
      py::object o = pyargs[i];
      Arg a;
      if (py::isinstance<py::tuple>(o) && py::len(o) == 2 && py::isinstance<py::str>(o.cast<py::tuple>()[0])) {
        auto t = o.cast<py::tuple>();
        std::string tag = t[0].cast<std::string>();
        if (tag == "slot") {
          a.kind = Arg::SLOT;
          a.slot = t[1].cast<int>();
        } else if (tag == "slots") {
          a.kind = Arg::SLOT_LIST;
          for (auto h : t[1].cast<py::list>()) a.slots.push_back(h.is_none() ? -1 : h.cast<int>());
          a.optional_list = schema.arguments()[i].type()->str().find("Tensor?[]") != std::string::npos;
        } else if (tag == "const") {
          a.kind = Arg::CONST;
          py::object v = t[1];
          const auto& ty = schema.arguments()[i].type();
          bool number = py::isinstance<py::bool_>(v) || py::isinstance<py::int_>(v) || py::isinstance<py::float_>(v);
          if (number && ty->kind() == c10::TypeKind::TensorType) {
            // a Python number in a Tensor position: a wrapped 0-dim tensor, as the Python dispatcher would pass
            c10::Scalar sc = py::isinstance<py::bool_>(v)  ? c10::Scalar(v.cast<bool>())
                             : py::isinstance<py::int_>(v) ? c10::Scalar(v.cast<int64_t>())
                                                           : c10::Scalar(v.cast<double>());
            at::Tensor w = c10::scalar_to_tensor(sc);
            w.unsafeGetTensorImpl()->set_wrapped_number(true);
            a.value = w;
          } else {
            a.value = torch::jit::toIValue(v, ty);
          }
        } else {
          TORCH_CHECK(false, "unknown argument tag ", tag);
        }
      } else {
        TORCH_CHECK(false, name, ": arguments must be tagged tuples");
      }
      in.args.push_back(std::move(a));
    }
    in.out_slots = {out_slot};
    in.free_after = std::move(free_after);
    prog.push_back(std::move(in));
    return (int)prog.size() - 1;
  }

  int add_fused(std::shared_ptr<jit::Kernel> k, std::vector<int> in_slots, std::vector<int64_t> out_shape,
                std::vector<at::ScalarType> out_dtypes, std::vector<int> out_slots, int vec,
                std::vector<int> free_after, const std::string& name) {
    TORCH_CHECK(in_slots.size() + out_slots.size() <= (size_t)jit::kMaxOperands, "too many operands in ", name);
    TORCH_CHECK(out_shape.size() <= (size_t)jit::kMaxDims, "too many dimensions in ", name);
    Instr in;
    in.kind = Instr::FUSED;
    in.name = name;
    in.kernel = std::move(k);
    in.in_slots = std::move(in_slots);
    in.out_shape = std::move(out_shape);
    in.out_dtypes = std::move(out_dtypes);
    in.out_slots = std::move(out_slots);
    in.vec = vec;
    in.free_after = std::move(free_after);
    prog.push_back(std::move(in));
    return (int)prog.size() - 1;
  }

  int add_getitem(int src, int index, int out_slot, std::vector<int> free_after) {
    Instr in;
    in.kind = Instr::GETITEM;
    in.src = src;
    in.index = index;
    in.out_slots = {out_slot};
    in.free_after = std::move(free_after);
    prog.push_back(std::move(in));
    return (int)prog.size() - 1;
  }

  std::vector<c10::IValue> run(std::vector<c10::IValue> inputs) {
    TORCH_CHECK(inputs.size() == input_slots.size(), "graph expects ", input_slots.size(), " inputs, got ",
                inputs.size());
    std::vector<c10::IValue> slots(n_slots);
    for (size_t i = 0; i < inputs.size(); ++i)
      if (input_slots[i] >= 0) slots[input_slots[i]] = std::move(inputs[i]);
    inputs.clear();
    torch::jit::Stack stack;
    for (Instr& in : prog) {
      switch (in.kind) {
        case Instr::OP: run_op(in, slots, stack); break;
        case Instr::FUSED: run_fused(in, slots); break;
        case Instr::GETITEM: {
          const c10::IValue& s = slots[in.src];
          if (s.isTuple()) slots[in.out_slots[0]] = s.toTupleRef().elements()[in.index];
          else if (s.isList()) slots[in.out_slots[0]] = s.toListRef()[in.index];
          else TORCH_CHECK(false, "getitem on a value that is neither tuple nor list");
          break;
        }
      }
      for (int f : in.free_after) slots[f] = c10::IValue();
    }
    std::vector<c10::IValue> out;
    out.reserve(output_slots.size());
    for (int s : output_slots) out.push_back(s < 0 ? c10::IValue() : slots[s]);
    ++runs;
    return out;
  }

 private:
  void run_op(Instr& in, std::vector<c10::IValue>& slots, torch::jit::Stack& stack) {
    stack.clear();
    for (const Arg& a : in.args) {
      switch (a.kind) {
        case Arg::CONST: stack.push_back(a.value); break;
        case Arg::SLOT: stack.push_back(slots[a.slot]); break;
        case Arg::SLOT_LIST:
          if (a.optional_list) {
            c10::List<std::optional<at::Tensor>> l;
            for (int s : a.slots) l.push_back(s < 0 ? std::optional<at::Tensor>() : std::optional<at::Tensor>(slots[s].toTensor()));
            stack.emplace_back(std::move(l));
          } else {
            c10::List<at::Tensor> l;
            for (int s : a.slots) l.push_back(slots[s].toTensor());
            stack.emplace_back(std::move(l));
          }
          break;
      }
    }
    in.op->callBoxed(stack);
    ++op_calls;
    if (in.out_slots[0] >= 0) {
      if (stack.size() == 1) slots[in.out_slots[0]] = std::move(stack[0]);
      else if (stack.size() > 1) slots[in.out_slots[0]] = c10::ivalue::Tuple::create(std::move(stack));
    }
    stack.clear();
  }

  void run_fused(Instr& in, std::vector<c10::IValue>& slots) {
    jit::PointwiseArgs pa{};
    const int nd = (int)in.out_shape.size();
    pa.ndim = nd;
    int64_t numel = 1;
    for (int d = 0; d < nd; ++d) {
      pa.sizes[d] = (int)in.out_shape[d];
      numel *= in.out_shape[d];
    }
    pa.numel = numel;
    const int ni = (int)in.in_slots.size();
    bool fast = in.vec > 1 && numel % in.vec == 0;
    // Fast-path addressing per operand: {period, divisor}.  period 0 = one element for everything; period P =
    // element (i mod P) (P = numel: dense; P < numel: a dense operand that spans the trailing dimensions);
    // divisor D > 0 = element (i / D) (a dense operand that spans the leading dimensions, e.g. one value per row).
    long long fast_mode[jit::kMaxOperands][2] = {};
    at::Tensor first;
    for (int i = 0; i < ni; ++i) {
      const at::Tensor& t = slots[in.in_slots[i]].toTensor();
      if (i == 0) first = t;
      pa.ptr[i] = t.data_ptr();
      const int td = (int)t.dim();
      TORCH_CHECK(td <= nd, in.name, ": operand rank exceeds the output rank");
      for (int d = 0; d < nd; ++d) {
        int sd = d - (nd - td);
        long long st = 0;
        if (sd >= 0 && t.size(sd) != 1) {
          TORCH_CHECK(t.size(sd) == in.out_shape[d], in.name, ": operand shape changed since compilation");
          st = t.stride(sd);
        }
        pa.strides[i][d] = st;
      }
      if (!fast) continue;
      const int64_t tn = t.numel();
      const bool aligned = (reinterpret_cast<uintptr_t>(pa.ptr[i]) & 15) == 0;
      if (tn == 1) {
        fast_mode[i][0] = 0;
      } else if (!t.is_contiguous()) {
        fast = false;
      } else if (tn == numel) {
        fast_mode[i][0] = numel;
        fast = fast && aligned;
      } else {
        // where do the operand's non-broadcast dimensions sit?
        int lo = nd, hi = -1;
        for (int d = 0; d < nd; ++d)
          if (pa.strides[i][d] != 0) { lo = std::min(lo, d); hi = std::max(hi, d); }
        int64_t span = 1, inner = 1;
        for (int d = lo; d <= hi; ++d) span *= in.out_shape[d];
        for (int d = hi + 1; d < nd; ++d) inner *= in.out_shape[d];
        if (span != tn) {
          fast = false;  // broadcast dimensions in the middle
        } else if (hi == nd - 1 && tn % in.vec == 0 && aligned) {
          fast_mode[i][0] = tn;
        } else if (lo == 0 && inner % in.vec == 0) {
          fast_mode[i][0] = numel;
          fast_mode[i][1] = inner;
        } else {
          fast = false;
        }
      }
    }
    if (fast)
      for (int i = 0; i < ni; ++i) {
        pa.strides[i][0] = fast_mode[i][0];
        pa.strides[i][1] = fast_mode[i][1];
      }
    TORCH_CHECK(ni > 0, in.name, ": fused kernel without tensor inputs");
    for (size_t o = 0; o < in.out_slots.size(); ++o) {
      at::Tensor out = at::empty(in.out_shape, first.options().dtype(in.out_dtypes[o]));
      pa.ptr[ni + o] = out.data_ptr();
      long long st = 1;
      for (int d = nd - 1; d >= 0; --d) {
        pa.strides[ni + o][d] = st;
        st *= in.out_shape[d];
      }
      slots[in.out_slots[o]] = std::move(out);
    }
    if (numel == 0) return;
    int use_fast = fast ? 1 : 0;
    int64_t per_thread = fast ? in.vec : 1;
    int64_t threads = (numel + per_thread - 1) / per_thread;
    unsigned grid = (unsigned)std::min<int64_t>((threads + 255) / 256, 148 * 16);
    void* params[] = {&pa, &use_fast};
    DeviceSwitch sw(first.device().index());
    in.kernel->launch(dim3(grid), dim3(256), 0, get_current_stream(first.device().index()).stream(), params);
    ++fused_launches;
  }
};

}  // namespace

void init_compile_bindings(py::module& m) {
  m.def("_storage_use_count", [](const at::Tensor& t) {
    // how many tensors / storages objects reference this memory (graph trees decide liveness from it)
    return (int64_t)t.storage().use_count();
  });
  m.def("_jit_available", [] {
    std::string why;
    bool ok = jit::compiler_available(&why);
    return py::make_tuple(ok, why);
  });
  py::class_<jit::Kernel, std::shared_ptr<jit::Kernel>>(m, "_JitKernel")
      .def(py::init([](const std::string& source, const std::string& entry) {
        return std::make_shared<jit::Kernel>(jit::compile_to_cubin(source, entry), entry);
      }))
      .def_static("from_cubin", [](py::bytes cubin, const std::string& entry) {
        return std::make_shared<jit::Kernel>(std::string(cubin), entry);
      })
      .def_property_readonly("cubin", [](jit::Kernel& k) { return py::bytes(k.cubin()); })
      .def_property_readonly("entry", &jit::Kernel::entry);

  py::class_<GraphRunner, std::shared_ptr<GraphRunner>>(m, "_GraphRunner")
      .def(py::init<>())
      .def_readwrite("n_slots", &GraphRunner::n_slots)
      .def_readwrite("input_slots", &GraphRunner::input_slots)
      .def_readwrite("output_slots", &GraphRunner::output_slots)
      .def_readonly("runs", &GraphRunner::runs)
      .def_readonly("fused_launches", &GraphRunner::fused_launches)
      .def_readonly("op_calls", &GraphRunner::op_calls)
      .def("__len__", [](GraphRunner& g) { return g.prog.size(); })
      .def("add_op", &GraphRunner::add_op, py::arg("name"), py::arg("overload"), py::arg("args"), py::arg("out_slot"),
           py::arg("free_after"), py::arg("label") = "")
      .def("add_fused", &GraphRunner::add_fused, py::arg("kernel"), py::arg("in_slots"), py::arg("out_shape"),
           py::arg("out_dtypes"), py::arg("out_slots"), py::arg("vec"), py::arg("free_after"), py::arg("label") = "")
      .def("add_getitem", &GraphRunner::add_getitem)
      .def("run", [](GraphRunner& g, py::list args) {
        std::vector<c10::IValue> in;
        in.reserve(args.size());
        for (auto h : args) {
          if (h.is_none()) in.emplace_back();
          else if (THPVariable_Check(h.ptr())) in.emplace_back(THPVariable_Unpack(h.ptr()));
          else if (py::isinstance<py::bool_>(h)) in.emplace_back(h.cast<bool>());
          else if (py::isinstance<py::int_>(h)) in.emplace_back(h.cast<int64_t>());
          else if (py::isinstance<py::float_>(h)) in.emplace_back(h.cast<double>());
          else TORCH_CHECK(false, "graph inputs must be tensors, numbers or None");
        }
        std::vector<c10::IValue> out;
        {
          py::gil_scoped_release nogil;
          out = g.run(std::move(in));
        }
        py::list res;
        for (auto& v : out) res.append(torch::jit::toPyObject(std::move(v)));
        return res;
      });
}

}  // namespace b200
