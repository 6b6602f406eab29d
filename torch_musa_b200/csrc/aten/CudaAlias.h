// Zero-copy bridge between blackwell (PrivateUse1) tensors and CUDA tensors.
//
// A blackwell tensor lives in ordinary CUDA device memory, so the long tail of
// operators that this backend does not implement by hand can run on PyTorch's
// own CUDA kernels without moving a byte: the boxed fallback re-labels every
// tensor argument as a CUDA tensor over the same storage, runs the op on the
// caller's blackwell stream, and re-labels the results.  The reference fills
// the same gap by text-porting ~120 of PyTorch's CUDA kernel files at build
// time (reference tools/cuda_porting/cuda_porting.py:81-229,
// torch_musa/csrc/CMakeLists.txt:58-184); re-using the kernels in place of
// re-compiling them needs no code generator and no patched torch.
// Hot-path operators never come here: they have explicit PrivateUse1 kernels.
#pragma once

#include "core/Device.h"

#include <ATen/core/Tensor.h>
#include <ATen/core/stack.h>
#include <c10/cuda/CUDAStream.h>

#include <vector>

namespace b200 {
namespace bridge {

// Per-call translation context: keeps one CUDA storage per blackwell storage so that
// arguments which alias each other still alias after translation.
class B200_EXPORT AliasScope {
 public:
  // blackwell -> CUDA view of the same memory (other tensors pass through untouched)
  at::Tensor to_cuda(const at::Tensor& t);
  // CUDA result -> blackwell tensor. Results that share storage with a translated argument become
  // views of the original blackwell storage; fresh results wrap (and keep alive) the CUDA storage.
  at::Tensor from_cuda(const at::Tensor& t);
  // After the op ran: propagate resizes of translated `out=`/in-place arguments back to the originals.
  void sync_back();

 private:
  struct Entry {
    at::Tensor orig;
    at::Tensor alias;
    const void* data_before;
  };
  struct StoragePair {
    c10::StorageImpl* orig;
    c10::Storage alias;
    c10::Storage orig_storage;
  };
  std::vector<Entry> tensors_;
  std::vector<StoragePair> storages_;
};

// A storage over the same bytes as `s`, labelled with device `dev`; `s` stays alive as long as the result.
B200_EXPORT c10::Storage relabel_storage(const c10::Storage& s, c10::Device dev);
// Wraps CUDA memory owned by `cuda_storage` as a blackwell storage (keeps it alive).
B200_EXPORT c10::Storage wrap_cuda_storage(const c10::Storage& cuda_storage);
// True if the DataPtr was produced by wrap_cuda_storage; optionally returns the wrapped CUDA storage.
B200_EXPORT bool is_wrapped_cuda(const c10::DataPtr& p, c10::Storage* out = nullptr);

// RAII: makes torch's current CUDA stream equal to the current blackwell stream of `device`.
struct B200_EXPORT CudaStreamMirror {
  explicit CudaStreamMirror(c10::DeviceIndex device);
  ~CudaStreamMirror();
 private:
  c10::cuda::CUDAStream prev_;
  c10::DeviceIndex device_;
};

// The boxed fallback itself.
B200_EXPORT void cuda_alias_fallback(const c10::OperatorHandle& op, torch::jit::Stack* stack);

// Names of operators that went through the fallback (for coverage reports), with call counts.
B200_EXPORT std::vector<std::pair<std::string, int64_t>> fallback_counts();
B200_EXPORT void reset_fallback_counts();
B200_EXPORT void set_fallback_logging(int level);  // 0 silent, 1 count, 2 warn once per op

// Convenience for hand-written ops that want to delegate a rare configuration to the CUDA kernel.
template <class F>
auto with_cuda(c10::DeviceIndex device, F&& f) {
  CudaStreamMirror m(device);
  return f();
}

}  // namespace bridge
}  // namespace b200
