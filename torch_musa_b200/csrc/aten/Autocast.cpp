// Autocast policy for the blackwell device: which operators run in the low-precision
// dtype, which are forced to fp32 and which promote to the widest input.  The lists
// are the framework's own (shared with its CUDA backend), so a model autocasts the
// same way on both; this backend's fused ops are added to the matching class.
// Parity: reference torch_musa/csrc/amp/autocast_mode.cpp:24-76.
#include <ATen/autocast_mode.h>
#include <torch/library.h>

namespace {
using namespace at::autocast;

at::Tensor bce_banned(const at::Tensor&, const at::Tensor&, const std::optional<at::Tensor>&, int64_t) {
  TORCH_CHECK(false,
              "torch.nn.functional.binary_cross_entropy and torch.nn.BCELoss are unsafe to autocast.\n"
              "Use torch.nn.functional.binary_cross_entropy_with_logits or torch.nn.BCEWithLogitsLoss, which "
              "combine the sigmoid and the loss and are safe to autocast.");
}

// Operators without an autocast rule pass through untouched.
TORCH_LIBRARY_IMPL(_, AutocastPrivateUse1, m) { m.fallback(torch::CppFunction::makeFallthrough()); }

TORCH_LIBRARY_IMPL(aten, AutocastPrivateUse1, m) {
#define _KERNEL_PU1_LOW_PRECISION_FP(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, lower_precision_fp)
  AT_FORALL_LOWER_PRECISION_FP(_KERNEL_PU1_LOW_PRECISION_FP)
#undef _KERNEL_PU1_LOW_PRECISION_FP

#define _KERNEL_PU1_FP32(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, fp32)
  AT_FORALL_FP32(_KERNEL_PU1_FP32)
#undef _KERNEL_PU1_FP32

#define _KERNEL_PU1_FP32_SET_OPT_DTYPE(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, fp32_set_opt_dtype)
  AT_FORALL_FP32_SET_OPT_DTYPE(_KERNEL_PU1_FP32_SET_OPT_DTYPE)
#undef _KERNEL_PU1_FP32_SET_OPT_DTYPE

#define _KERNEL_PU1_PROMOTE(...) KERNEL_PRIVATEUSEONE(__VA_ARGS__, promote)
  AT_FORALL_PROMOTE(_KERNEL_PU1_PROMOTE)
#undef _KERNEL_PU1_PROMOTE

  m.impl(TORCH_SELECTIVE_NAME("aten::binary_cross_entropy"), TORCH_FN(bce_banned));
}

// The backend's own fused ops (RoPE, SwiGLU, fused cross entropy) have no autocast kernel on purpose:
// the framework-wide AutocastPrivateUse1 fallthrough applies, so they follow their input dtype -- they
// sit between autocast GEMMs -- and accumulate in fp32 internally.

}  // namespace
