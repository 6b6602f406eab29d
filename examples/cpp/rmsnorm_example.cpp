// Using the kernel library (libb200_kernels.so) from plain C++, without Python or libtorch: allocate with the CUDA
// runtime, call the C ABI of b200_kernels.h, compare with a host reference.
//
//   make -C examples/cpp && ./examples/cpp/rmsnorm_example
//
// (The reference ships a libtorch-based C++ example: reference examples/cpp/.)
#include "b200_kernels.h"

#include <cuda_runtime_api.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#define CHECK(x)                                                                  \
  do {                                                                            \
    int e_ = (int)(x);                                                            \
    if (e_ != 0) {                                                                \
      std::fprintf(stderr, "%s failed: %s\n", #x, cudaGetErrorString((cudaError_t)e_)); \
      return 1;                                                                   \
    }                                                                             \
  } while (0)

int main() {
  const int64_t rows = 512, cols = 4096;
  const float eps = 1e-5f;
  std::printf("kernel library built for %s\n", b200_kernels_arch());
  std::vector<float> hx(rows * cols), hw(cols);
  for (size_t i = 0; i < hx.size(); ++i) hx[i] = (float)((i * 2654435761u) % 2001) / 1000.f - 1.f;
  for (int64_t c = 0; c < cols; ++c) hw[c] = 0.5f + (float)(c % 7) * 0.1f;
  float *x = nullptr, *w = nullptr, *y = nullptr, *rstd = nullptr;
  CHECK(cudaMalloc((void**)&x, hx.size() * sizeof(float)));
  CHECK(cudaMalloc((void**)&w, hw.size() * sizeof(float)));
  CHECK(cudaMalloc((void**)&y, hx.size() * sizeof(float)));
  CHECK(cudaMalloc((void**)&rstd, rows * sizeof(float)));
  CHECK(cudaMemcpy(x, hx.data(), hx.size() * sizeof(float), cudaMemcpyHostToDevice));
  CHECK(cudaMemcpy(w, hw.data(), hw.size() * sizeof(float), cudaMemcpyHostToDevice));
  cudaStream_t stream;
  CHECK(cudaStreamCreate(&stream));
  CHECK(b200_rmsnorm_fwd(B200_F32, y, rstd, x, w, /*residual=*/nullptr, /*res_out=*/nullptr, rows, cols, eps, stream));
  CHECK(cudaStreamSynchronize(stream));
  std::vector<float> hy(hx.size());
  CHECK(cudaMemcpy(hy.data(), y, hy.size() * sizeof(float), cudaMemcpyDeviceToHost));
  double worst = 0.0;
  for (int64_t r = 0; r < rows; ++r) {
    double ss = 0.0;
    for (int64_t c = 0; c < cols; ++c) ss += (double)hx[r * cols + c] * hx[r * cols + c];
    const double rs = 1.0 / std::sqrt(ss / cols + eps);
    for (int64_t c = 0; c < cols; ++c)
      worst = std::fmax(worst, std::fabs(hx[r * cols + c] * rs * hw[c] - hy[r * cols + c]));
  }
  std::printf("rmsnorm [%lld x %lld]: max abs error %.3g, own kernel launches %lld\n", (long long)rows, (long long)cols,
              worst, (long long)b200_launch_count());
  cudaFree(x); cudaFree(w); cudaFree(y); cudaFree(rstd);
  cudaStreamDestroy(stream);
  return worst < 1e-4 ? 0 : 2;
}
