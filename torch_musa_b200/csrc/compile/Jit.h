// Run-time compilation of generated CUDA C++ (NVRTC -> sm_100a cubin -> cudaLibrary) for the
// compile stack's fused pointwise kernels.  The compiler library is opened with dlopen, so the
// package imports and compiles on machines without a GPU; only load()/launch() need a device.
#pragma once

#include "core/Device.h"

#include <cuda_runtime.h>

#include <memory>
#include <string>
#include <vector>

namespace b200 {
namespace jit {

// Compiles `source` for sm_100a and returns the cubin image.  Throws with the compiler log on error.
B200_EXPORT std::string compile_to_cubin(const std::string& source, const std::string& name,
                                        const std::vector<std::string>& extra_options = {});
B200_EXPORT bool compiler_available(std::string* why = nullptr);

// Argument block every generated pointwise kernel takes by value.
constexpr int kMaxOperands = 12;
constexpr int kMaxDims = 6;
struct PointwiseArgs {
  void* ptr[kMaxOperands];               // inputs first, then outputs
  long long numel;                       // of the (broadcast) output shape
  int ndim;
  int sizes[kMaxDims];                   // output shape, outermost first
  long long strides[kMaxOperands][kMaxDims];  // element strides against the output shape (0 = broadcast)
};

class B200_EXPORT Kernel {
 public:
  Kernel(std::string cubin, std::string entry);
  ~Kernel();
  Kernel(const Kernel&) = delete;
  // Loads on first use for the current device.
  void launch(dim3 grid, dim3 block, size_t smem, cudaStream_t stream, void** params);
  const std::string& entry() const { return entry_; }
  const std::string& cubin() const { return cubin_; }

 private:
  std::string cubin_, entry_;
  struct PerDevice { cudaLibrary_t lib = nullptr; cudaKernel_t fn = nullptr; };
  std::vector<PerDevice> dev_;
};

}  // namespace jit
}  // namespace b200
