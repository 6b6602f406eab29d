#include "compile/Jit.h"

#include <c10/util/Exception.h>

#include <dlfcn.h>

#include <mutex>

namespace b200 {
namespace jit {
namespace {

// The handful of NVRTC entry points, resolved by name (no header or link dependency on the library).
struct Nvrtc {
  using Program = void*;
  int (*create)(Program*, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
  int (*destroy)(Program*) = nullptr;
  int (*compile)(Program, int, const char* const*) = nullptr;
  int (*log_size)(Program, size_t*) = nullptr;
  int (*log)(Program, char*) = nullptr;
  int (*cubin_size)(Program, size_t*) = nullptr;
  int (*cubin)(Program, char*) = nullptr;
  const char* (*error_string)(int) = nullptr;
  std::string why;
  bool ok = false;
};

const Nvrtc& nvrtc() {
  static Nvrtc n = [] {
    Nvrtc v;
    const char* names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12",
                           "/usr/local/cuda/lib64/libnvrtc.so"};
    void* h = nullptr;
    if (const char* env = std::getenv("B200_NVRTC_PATH")) h = dlopen(env, RTLD_NOW | RTLD_LOCAL);
    for (const char* nm : names) {
      if (h) break;
      h = dlopen(nm, RTLD_NOW | RTLD_LOCAL);
    }
    if (!h) {
      v.why = "libnvrtc.so.12 not found (set B200_NVRTC_PATH)";
      return v;
    }
    auto sym = [&](const char* s, void** out) {
      *out = dlsym(h, s);
      return *out != nullptr;
    };
    v.ok = sym("nvrtcCreateProgram", (void**)&v.create) && sym("nvrtcDestroyProgram", (void**)&v.destroy) &&
           sym("nvrtcCompileProgram", (void**)&v.compile) && sym("nvrtcGetProgramLogSize", (void**)&v.log_size) &&
           sym("nvrtcGetProgramLog", (void**)&v.log) && sym("nvrtcGetCUBINSize", (void**)&v.cubin_size) &&
           sym("nvrtcGetCUBIN", (void**)&v.cubin) && sym("nvrtcGetErrorString", (void**)&v.error_string);
    if (!v.ok) v.why = "libnvrtc lacks an expected entry point";
    return v;
  }();
  return n;
}

}  // namespace

bool compiler_available(std::string* why) {
  const Nvrtc& n = nvrtc();
  if (!n.ok && why) *why = n.why;
  return n.ok;
}

std::string compile_to_cubin(const std::string& source, const std::string& name,
                             const std::vector<std::string>& extra) {
  const Nvrtc& n = nvrtc();
  TORCH_CHECK(n.ok, "run-time kernel compiler unavailable: ", n.why);
  Nvrtc::Program prog = nullptr;
  int e = n.create(&prog, source.c_str(), (name + ".cu").c_str(), 0, nullptr, nullptr);
  TORCH_CHECK(e == 0, "nvrtcCreateProgram: ", n.error_string(e));
  // No fast-math: fused results must match the unfused operators.  Generated sources include no headers.
  std::vector<std::string> opts = {"--gpu-architecture=sm_100a", "--std=c++17", "-default-device"};
  for (auto& o : extra) opts.push_back(o);
  std::vector<const char*> copts;
  for (auto& o : opts) copts.push_back(o.c_str());
  e = n.compile(prog, (int)copts.size(), copts.data());
  if (e != 0) {
    size_t ls = 0;
    n.log_size(prog, &ls);
    std::string log(ls, '\0');
    if (ls) n.log(prog, log.data());
    n.destroy(&prog);
    TORCH_CHECK(false, "compiling generated kernel '", name, "' failed: ", n.error_string(e), "\n", log);
  }
  size_t cs = 0;
  n.cubin_size(prog, &cs);
  std::string cubin(cs, '\0');
  n.cubin(prog, cubin.data());
  n.destroy(&prog);
  TORCH_CHECK(cs > 0, "the compiler produced no cubin for '", name, "'");
  return cubin;
}

Kernel::Kernel(std::string cubin, std::string entry) : cubin_(std::move(cubin)), entry_(std::move(entry)) {}

Kernel::~Kernel() {
  for (auto& d : dev_)
    if (d.lib) (void)cudaLibraryUnload(d.lib);
}

void Kernel::launch(dim3 grid, dim3 block, size_t smem, cudaStream_t stream, void** params) {
  int device = 0;
  B200_CUDA_CHECK(cudaGetDevice(&device));
  static std::mutex mu;
  {
    std::lock_guard<std::mutex> g(mu);
    if ((int)dev_.size() <= device) dev_.resize(device + 1);
    if (!dev_[device].fn) {
      B200_CUDA_CHECK(cudaLibraryLoadData(&dev_[device].lib, cubin_.data(), nullptr, nullptr, 0, nullptr, nullptr, 0));
      B200_CUDA_CHECK(cudaLibraryGetKernel(&dev_[device].fn, dev_[device].lib, entry_.c_str()));
    }
  }
  B200_CUDA_CHECK(cudaLaunchKernel((const void*)dev_[device].fn, grid, block, params, smem, stream));
}

}  // namespace jit
}  // namespace b200
