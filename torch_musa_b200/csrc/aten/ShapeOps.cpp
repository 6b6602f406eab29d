// Concatenation operators on the hand-written copy kernels.
//
// `cat` writes every input into its slice of the output with one row-vectorised copy (16-byte accesses,
// dtype conversion in flight); `_chunk_cat` -- the copy-in of FSDP2's gradient reduce-scatter: every
// gradient is cut into world_size chunks and chunk r of every gradient is packed into row r of the
// output, usually converting bf16 to the fp32 reduce dtype -- is the same copy with a two-row stride
// pattern.  Without these the composite implementations run per-element strided kernels that are an
// order of magnitude slower on 100 MB-sized gradients.
// Parity: reference torch_musa/csrc/aten/ops/Cat.cpp, and the FSDP2 copy-in patch
// torch_musa/distributed/_composable/fsdp/patch.py:60-123.
#include "aten/FallbackCall.h"
#include "aten/Ops.h"

#include <ATen/Functions.h>
#include <ATen/NativeFunctions.h>
#include <ATen/WrapDimUtils.h>
#include <torch/library.h>

namespace b200 {
namespace ops {

namespace {

bool legacy_skip(const at::Tensor& t) { return t.dim() == 1 && t.numel() == 0; }

bool cat_native_ok(const at::ITensorListRef& tensors, const at::Tensor& out) {
  // any element type: pieces of a type the cast-copy kernel does not know go through copy_ (a device-side
  // strided copy as well), e.g. the int64 step counters that DistributedDataParallel flattens every step
  if (!on_device(out)) return false;
  for (const at::Tensor& t : tensors) {
    if (!on_device(t) || t.device() != out.device()) return false;
    if (t.is_conj() || t.is_neg()) return false;
  }
  return true;
}

at::Tensor& cat_out(const at::ITensorListRef& tensors, int64_t dim, at::Tensor& out) {
  const at::Tensor* first = nullptr;
  for (const at::Tensor& t : tensors)
    if (!legacy_skip(t)) { first = &t; break; }
  bool native = first != nullptr && cat_native_ok(tensors, out);
  if (native) {
    // only the plain case: no dtype promotion among the inputs, output dtype as given
    for (const at::Tensor& t : tensors)
      if (!legacy_skip(t) && (t.scalar_type() != first->scalar_type() || t.dim() != first->dim())) native = false;
  }
  if (!native) {
    std::vector<at::Tensor> v;
    for (const at::Tensor& t : tensors) v.push_back(t);
    run_fallback(B200_OP_HANDLE("aten::cat", "out"), v, dim, out);
    return out;
  }
  const int64_t nd = first->dim();
  const int64_t d = at::maybe_wrap_dim(dim, nd);
  std::vector<int64_t> shape = first->sizes().vec();
  int64_t total = 0;
  for (const at::Tensor& t : tensors) {
    if (legacy_skip(t)) continue;
    for (int64_t i = 0; i < nd; ++i)
      TORCH_CHECK(i == d || t.size(i) == shape[i], "Sizes of tensors must match except in dimension ", d,
                  ". Expected size ", shape[i], " but got size ", t.size(i), " for a tensor in the list.");
    total += t.size(d);
  }
  shape[d] = total;
  if (out.sizes() != at::IntArrayRef(shape)) out.resize_(shape);
  if (out.numel() == 0) return out;
  auto stream = current_raw_stream(out);
  // outermost-dimension concatenation of contiguous pieces of the output's type: one byte-copy launch per 128 pieces
  int64_t outer = 1;
  for (int64_t i = 0; i < d; ++i) outer *= shape[i];
  bool bytes_ok = outer == 1 && out.is_contiguous() && out.scalar_type() == first->scalar_type();
  if (bytes_ok)
    for (const at::Tensor& t : tensors)
      if (!legacy_skip(t) && !t.is_contiguous()) bytes_ok = false;
  if (bytes_ok) {
    std::vector<const void*> srcs;
    std::vector<int64_t> nbytes;
    for (const at::Tensor& t : tensors) {
      if (legacy_skip(t) || t.numel() == 0) continue;
      srcs.push_back(t.const_data_ptr());
      nbytes.push_back((int64_t)t.numel() * (int64_t)t.element_size());
    }
    DeviceSwitch sw(out.device().index());
    B200_KERNEL_CALL(b200_cat_bytes(out.mutable_data_ptr(), srcs.data(), nbytes.data(), (int)srcs.size(), stream));
    return out;
  }
  int64_t off = 0;
  for (const at::Tensor& t : tensors) {
    if (legacy_skip(t) || t.size(d) == 0) continue;
    at::Tensor dst = out.narrow(d, off, t.size(d));
    if (!try_native_cast_copy(t, dst, stream)) dst.copy_(t);
    off += t.size(d);
  }
  return out;
}

at::Tensor cat(const at::ITensorListRef& tensors, int64_t dim) {
  const at::Tensor* first = nullptr;
  for (const at::Tensor& t : tensors)
    if (!legacy_skip(t)) { first = &t; break; }
  bool plain_case = first != nullptr && on_device(*first);
  if (plain_case)
    for (const at::Tensor& t : tensors)
      if (!legacy_skip(t) && (t.scalar_type() != first->scalar_type() || !on_device(t))) plain_case = false;
  if (!plain_case) {
    std::vector<at::Tensor> v;
    for (const at::Tensor& t : tensors) v.push_back(t);
    return fallback_tensor(B200_OP_HANDLE("aten::cat", ""), v, dim);
  }
  at::Tensor out = at::empty({0}, first->options());
  return cat_out(tensors, dim, out);
}

// out[r, off_i : off_i + cols_i] = chunk r of tensor i (flattened), zero padded where a tensor's first
// dimension does not divide evenly.
at::Tensor& chunk_cat_out(at::TensorList tensors, int64_t dim, int64_t num_chunks, at::Tensor& out) {
  bool native = dim == 0 && num_chunks >= 1 && on_device(out) && kdtype(out.scalar_type()) >= 0 && out.dim() == 2 &&
                out.is_contiguous() && !tensors.empty();
  int64_t cols = 0;
  if (native) {
    for (const at::Tensor& t : tensors) {
      if (!on_device(t) || kdtype(t.scalar_type()) < 0 || t.dim() < 1 || t.size(0) == 0 || !t.is_contiguous()) {
        native = false;
        break;
      }
      const int64_t rows = (t.size(0) + num_chunks - 1) / num_chunks;
      cols += rows * (t.numel() / t.size(0));
    }
  }
  if (!native || out.size(0) != num_chunks || out.size(1) != cols) return at::native::_chunk_cat_out(tensors, dim, num_chunks, out);
  auto stream = current_raw_stream(out);
  int64_t off = 0;
  for (const at::Tensor& t : tensors) {
    const int64_t rest = t.numel() / t.size(0);
    const int64_t rows = (t.size(0) + num_chunks - 1) / num_chunks;
    const int64_t width = rows * rest;
    const int64_t full = t.size(0) / rows;           // chunks that are completely filled
    const int64_t rem = t.size(0) - full * rows;     // rows in the partly filled chunk
    const at::Tensor flat = t.view({-1});
    if (full > 0) {
      at::Tensor src = flat.narrow(0, 0, full * width).view({full, width});
      at::Tensor dst = out.narrow(0, 0, full).narrow(1, off, width);
      if (!try_native_cast_copy(src, dst, stream)) dst.copy_(src);
    }
    if (full < num_chunks) {
      if (rem > 0) {
        at::Tensor src = flat.narrow(0, full * width, rem * rest).view({1, rem * rest});
        at::Tensor dst = out.narrow(0, full, 1).narrow(1, off, rem * rest);
        if (!try_native_cast_copy(src, dst, stream)) dst.copy_(src);
        out.narrow(0, full, 1).narrow(1, off + rem * rest, width - rem * rest).zero_();
      } else {
        out.narrow(0, full, 1).narrow(1, off, width).zero_();
      }
      if (full + 1 < num_chunks) out.narrow(0, full + 1, num_chunks - full - 1).narrow(1, off, width).zero_();
    }
    off += width;
  }
  return out;
}

at::Tensor chunk_cat(at::TensorList tensors, int64_t dim, int64_t num_chunks) {
  if (dim != 0 || tensors.empty() || !on_device(tensors[0]) || tensors[0].dim() < 1)
    return at::native::_chunk_cat(tensors, dim, num_chunks);
  int64_t cols = 0;
  for (const at::Tensor& t : tensors) {
    if (t.dim() < 1 || t.size(0) == 0 || t.scalar_type() != tensors[0].scalar_type())
      return at::native::_chunk_cat(tensors, dim, num_chunks);
    cols += ((t.size(0) + num_chunks - 1) / num_chunks) * (t.numel() / t.size(0));
  }
  at::Tensor out = at::empty({num_chunks, cols}, tensors[0].options());
  return chunk_cat_out(tensors, dim, num_chunks, out);
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("cat", TORCH_FN(cat));
  m.impl("cat.out", TORCH_FN(cat_out));
  m.impl("_chunk_cat", TORCH_FN(chunk_cat));
  m.impl("_chunk_cat.out", TORCH_FN(chunk_cat_out));
}

}  // namespace ops
}  // namespace b200
