// Concatenation along the outermost dimension of contiguous pieces of one element type: a byte copy of up to 128
// pieces per launch (pointer table in the kernel parameters), 16-byte vectors where source and destination allow.
// One launch replaces one copy per piece, which matters for the lists of tiny tensors that data-parallel wrappers
// flatten every step (step counters, bucket views).
// Parity: reference torch_musa/csrc/aten/ops/musa/TensorShape.mu (concatenation kernels).
#include "common.cuh"

namespace b200k {
namespace {

constexpr int kMaxPieces = 128;
constexpr int kChunkBytes = 1 << 16;

struct CatTable {
  const uint8_t* src[kMaxPieces];
  long long dst_off[kMaxPieces];
  long long nbytes[kMaxPieces];
};

__global__ void __launch_bounds__(256) cat_bytes_kernel(uint8_t* __restrict__ dst, const CatTable t) {
  const int piece = blockIdx.y;
  const long long n = t.nbytes[piece];
  const uint8_t* __restrict__ s = t.src[piece];
  uint8_t* __restrict__ d = dst + t.dst_off[piece];
  for (long long c0 = (long long)blockIdx.x * kChunkBytes; c0 < n; c0 += (long long)gridDim.x * kChunkBytes) {
    const long long len = min((long long)kChunkBytes, n - c0);
    const uint8_t* sp = s + c0;
    uint8_t* dp = d + c0;
    if (((reinterpret_cast<uintptr_t>(sp) | reinterpret_cast<uintptr_t>(dp)) & 15) == 0) {
      const long long v = len >> 4;
      for (long long i = threadIdx.x; i < v; i += blockDim.x)
        reinterpret_cast<uint4*>(dp)[i] = reinterpret_cast<const uint4*>(sp)[i];
      for (long long i = (v << 4) + threadIdx.x; i < len; i += blockDim.x) dp[i] = sp[i];
    } else {
      for (long long i = threadIdx.x; i < len; i += blockDim.x) dp[i] = sp[i];
    }
  }
}

}  // namespace
}  // namespace b200k

using namespace b200k;

extern "C" int b200_cat_bytes(void* dst, const void* const* srcs, const int64_t* nbytes, int n_pieces, cudaStream_t stream) {
  long long off = 0;
  for (int p0 = 0; p0 < n_pieces; p0 += kMaxPieces) {
    CatTable t;
    const int n = n_pieces - p0 < kMaxPieces ? n_pieces - p0 : kMaxPieces;
    long long longest = 0;
    for (int i = 0; i < n; ++i) {
      t.src[i] = static_cast<const uint8_t*>(srcs[p0 + i]);
      t.dst_off[i] = off;
      t.nbytes[i] = nbytes[p0 + i];
      off += nbytes[p0 + i];
      if (nbytes[p0 + i] > longest) longest = nbytes[p0 + i];
    }
    if (longest == 0) continue;
    long long gx = (longest + kChunkBytes - 1) / kChunkBytes;
    if (gx > 1184) gx = 1184;
    cat_bytes_kernel<<<dim3((unsigned)gx, (unsigned)n), 256, 0, stream>>>(static_cast<uint8_t*>(dst), t);
    ::b200k::note_launch();
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return (int)e;
  }
  return 0;
}
