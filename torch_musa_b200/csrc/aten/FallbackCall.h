// Helper for hand-written operators that cover only part of an op's domain: the rest is
// forwarded, boxed, to the CUDA-alias fallback (same memory, PyTorch's CUDA kernel).
#pragma once

#include "aten/CudaAlias.h"

#include <ATen/core/dispatch/Dispatcher.h>
#include <ATen/core/stack.h>

namespace b200 {
namespace ops {

template <class... Args>
inline torch::jit::Stack run_fallback(const c10::OperatorHandle& op, Args&&... args) {
  torch::jit::Stack stack;
  stack.reserve(sizeof...(Args));
  torch::jit::push(stack, std::forward<Args>(args)...);
  bridge::cuda_alias_fallback(op, &stack);
  return stack;
}

#define B200_OP_HANDLE(NAME, OVERLOAD)                                                        \
  ([]() -> const c10::OperatorHandle& {                                                       \
    static const c10::OperatorHandle h = c10::Dispatcher::singleton().findSchemaOrThrow(NAME, OVERLOAD); \
    return h;                                                                                 \
  }())

template <class... Args>
inline at::Tensor fallback_tensor(const c10::OperatorHandle& op, Args&&... args) {
  auto st = run_fallback(op, std::forward<Args>(args)...);
  return st.back().toTensor();
}

}  // namespace ops
}  // namespace b200
