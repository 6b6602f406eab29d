// The operators without which no tensor can exist on the device: allocation
// (empty / empty_strided), storage plumbing (resize_, set_), metadata-only
// views, host<->device and device<->device copies with dtype conversion,
// scalar read-back, record_stream and pinned-memory helpers.
// Parity: reference torch_musa/csrc/aten/ops/TensorFactory.cpp:33-162,331-424,
// Copy.cpp:179-260,336-470, Scalar.cpp, RecordStream.cpp:11-18.
#include "aten/CudaAlias.h"
#include "aten/Ops.h"
#include "core/Backend.h"
#include "core/CachingAllocator.h"
#include "core/HostAllocator.h"
#include "core/Stream.h"

#include <ATen/EmptyTensor.h>
#include <ATen/InferSize.h>
#include <ATen/NativeFunctions.h>
#include <ATen/native/Resize.h>
#include <ATen/ops/_copy_from_and_resize_native.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <torch/library.h>

namespace b200 {
namespace ops {

namespace {

constexpr c10::DispatchKeySet kKeys(c10::DispatchKey::PrivateUse1);

c10::DeviceIndex resolve_index(std::optional<c10::Device> d) {
  if (d.has_value() && d->has_index()) return d->index();
  return current_device();
}

at::Tensor empty_memory_format(c10::SymIntArrayRef size, std::optional<at::ScalarType> dtype,
                               std::optional<at::Layout> layout, std::optional<at::Device> device,
                               std::optional<bool> pin_memory, std::optional<at::MemoryFormat> mf) {
  TORCH_CHECK(!pin_memory.value_or(false), "Only dense CPU tensors can be pinned");
  TORCH_CHECK(layout.value_or(c10::kStrided) == c10::kStrided, "blackwell tensors must be strided");
  lazy_init();
  DeviceSwitch sw(resolve_index(device));
  return at::detail::empty_generic(C10_AS_INTARRAYREF_SLOW(size), c10::GetAllocator(kDeviceType), kKeys,
                                   c10::dtype_or_default(dtype), mf);
}

at::Tensor empty_strided(c10::SymIntArrayRef size, c10::SymIntArrayRef stride, std::optional<at::ScalarType> dtype,
                         std::optional<at::Layout> layout, std::optional<at::Device> device,
                         std::optional<bool> pin_memory) {
  TORCH_CHECK(!pin_memory.value_or(false), "Only dense CPU tensors can be pinned");
  lazy_init();
  DeviceSwitch sw(resolve_index(device));
  return at::detail::empty_strided_generic(C10_AS_INTARRAYREF_SLOW(size), C10_AS_INTARRAYREF_SLOW(stride),
                                           c10::GetAllocator(kDeviceType), kKeys, c10::dtype_or_default(dtype));
}

// ------------------------------------------------------------------ resize / set
void maybe_resize_storage(c10::TensorImpl* self, size_t new_bytes) {
  if (self->numel() == 0) return;
  const c10::Storage& storage = self->unsafe_storage();
  TORCH_CHECK(storage, "Tensor: invalid null storage");
  if (new_bytes > storage.nbytes()) resize_storage_bytes(storage.unsafeGetStorageImpl(), new_bytes);
}

const at::Tensor& resize_(const at::Tensor& self, c10::SymIntArrayRef size_, std::optional<at::MemoryFormat> mf) {
  auto size = C10_AS_INTARRAYREF_SLOW(size_);
  auto* impl = self.unsafeGetTensorImpl();
  if (impl->sizes() != size) {
    impl->set_sizes_contiguous(size);
    size_t bytes = (size_t)(impl->numel() + impl->storage_offset()) * impl->dtype().itemsize();
    maybe_resize_storage(impl, bytes);
  }
  if (mf.has_value() && *mf != at::MemoryFormat::Contiguous && *mf != at::MemoryFormat::Preserve) {
    impl->empty_tensor_restride(*mf);
  }
  return self;
}

at::Tensor& set_storage(at::Tensor& self, at::Storage source, c10::SymInt offset, c10::SymIntArrayRef size,
                        c10::SymIntArrayRef stride) {
  at::native::checkSetStorage(self, source, offset.expect_int(), C10_AS_INTARRAYREF_SLOW(size),
                              C10_AS_INTARRAYREF_SLOW(stride));
  auto* impl = self.unsafeGetTensorImpl();
  impl->set_storage_offset(offset.expect_int());
  auto sz = C10_AS_INTARRAYREF_SLOW(size);
  auto st = C10_AS_INTARRAYREF_SLOW(stride);
  if (st.data() != nullptr && st.size() == sz.size()) {
    impl->set_sizes_and_strides(sz, st);
  } else {
    impl->set_sizes_contiguous(sz);
  }
  size_t bytes = at::detail::computeStorageNbytes(impl->sizes(), impl->strides(), impl->dtype().itemsize(),
                                                  impl->storage_offset());
  maybe_resize_storage(impl, bytes);
  return self;
}

at::Tensor& set_source_storage(at::Tensor& self, at::Storage source) {
  int64_t n = (int64_t)(source.nbytes() / self.dtype().itemsize());
  c10::SymInt sn(n);
  return set_storage(self, std::move(source), 0, c10::SymIntArrayRef(&sn, 1), {});
}

at::Tensor& set_source_tensor(at::Tensor& self, const at::Tensor& source) {
  if (self.unsafeGetTensorImpl() != source.unsafeGetTensorImpl()) {
    return set_storage(self, source.storage(), source.sym_storage_offset(), source.sym_sizes(), source.sym_strides());
  }
  return self;
}

at::Tensor& set_empty(at::Tensor& self) {
  lazy_init();
  at::Storage st(c10::Storage::use_byte_size_t(), 0, c10::GetAllocator(kDeviceType), true);
  c10::SymInt zero(0);
  return set_storage(self, std::move(st), 0, c10::SymIntArrayRef(&zero, 1), {});
}

// ------------------------------------------------------------------ views
at::Tensor as_strided(const at::Tensor& self, c10::SymIntArrayRef size, c10::SymIntArrayRef stride,
                      std::optional<c10::SymInt> offset) {
  std::optional<int64_t> off;
  if (offset.has_value()) off = offset->expect_int();
  return at::native::as_strided_tensorimpl(self, C10_AS_INTARRAYREF_SLOW(size), C10_AS_INTARRAYREF_SLOW(stride), off);
}
at::Tensor view(const at::Tensor& self, c10::SymIntArrayRef size) {
  return at::native::view(self, C10_AS_INTARRAYREF_SLOW(size));
}
at::Tensor reshape_alias(const at::Tensor& self, c10::SymIntArrayRef size, c10::SymIntArrayRef stride) {
  return at::native::_reshape_alias(self, C10_AS_INTARRAYREF_SLOW(size), C10_AS_INTARRAYREF_SLOW(stride));
}
at::Tensor unfold(const at::Tensor& self, int64_t dim, int64_t size, int64_t step) {
  return at::native::unfold(self, dim, size, step);
}
at::Tensor view_as_real(const at::Tensor& self) { return at::native::view_as_real(self); }
at::Tensor view_as_complex(const at::Tensor& self) { return at::native::view_as_complex(self); }

// ------------------------------------------------------------------ copies
inline bool is_dev(const at::Tensor& t) { return t.device().type() == kDeviceType; }

bool same_dense_layout(const at::Tensor& a, const at::Tensor& b) {
  return a.sizes() == b.sizes() && a.strides() == b.strides() && a.is_non_overlapping_and_dense();
}

void copy_d2d(const at::Tensor& src, const at::Tensor& dst, bool non_blocking) {
  c10::DeviceIndex sd = src.device().index(), dd = dst.device().index();
  size_t nbytes = (size_t)src.numel() * src.dtype().itemsize();
  bool plain = src.dtype() == dst.dtype() && same_dense_layout(src, dst) && !src.is_conj() && !dst.is_conj() &&
               !src.is_neg() && !dst.is_neg();
  if (sd == dd) {
    DeviceSwitch sw(dd);
    cudaStream_t s = get_current_stream(dd).stream();
    if (plain) {
      if (nbytes && src.const_data_ptr() != dst.const_data_ptr())
        B200_CUDA_CHECK(cudaMemcpyAsync(dst.mutable_data_ptr(), src.const_data_ptr(), nbytes, cudaMemcpyDeviceToDevice, s));
      return;
    }
    if (try_native_cast_copy(src, dst, s)) return;
    bridge::AliasScope scope;
    bridge::CudaStreamMirror m(dd);
    scope.to_cuda(dst).copy_(scope.to_cuda(src), non_blocking);
    return;
  }
  // Cross-device: make the producer's work visible to the consumer's stream, copy on the destination stream,
  // and make the source stream wait so the source block is not recycled under the copy.
  bool p2p = enable_peer_access(dd, sd);
  (void)p2p;  // cudaMemcpyPeerAsync stages through the host when P2P is unavailable
  Stream src_stream = get_current_stream(sd), dst_stream = get_current_stream(dd);
  Event ready;
  ready.record(src_stream);
  ready.block(dst_stream);
  at::Tensor src_c = src;
  if (!plain) {
    // bring a contiguous, dtype-matched image over first, then scatter locally
    at::Tensor tmp_src = src.to(dst.scalar_type()).contiguous();
    Event r2;
    r2.record(src_stream);
    r2.block(dst_stream);
    at::Tensor tmp_dst;
    {
      DeviceSwitch sw(dd);
      tmp_dst = at::empty_like(tmp_src, tmp_src.options().device(dst.device()));
      B200_CUDA_CHECK(cudaMemcpyPeerAsync(tmp_dst.mutable_data_ptr(), dd, tmp_src.const_data_ptr(), sd,
                                          (size_t)tmp_src.numel() * tmp_src.dtype().itemsize(), dst_stream.stream()));
    }
    Event done;
    done.record(dst_stream);
    done.block(src_stream);
    alloc::get()->record_stream(tmp_src.storage().data_ptr(), dd, dst_stream.stream());
    copy_d2d(tmp_dst.expand_as(dst), dst, non_blocking);
    return;
  }
  {
    DeviceSwitch sw(dd);
    B200_CUDA_CHECK(cudaMemcpyPeerAsync(dst.mutable_data_ptr(), dd, src.const_data_ptr(), sd, nbytes, dst_stream.stream()));
  }
  Event done;
  done.record(dst_stream);
  done.block(src_stream);
}

void copy_h2d(const at::Tensor& src, const at::Tensor& dst, bool non_blocking) {
  c10::DeviceIndex dd = dst.device().index();
  DeviceSwitch sw(dd);
  Stream stream = get_current_stream(dd);
  bool direct = src.dtype() == dst.dtype() && src.is_contiguous() && dst.is_contiguous() && !src.is_conj() &&
                !src.is_neg();
  if (!direct) {
    bool dense_same = src.dtype() == dst.dtype() && same_dense_layout(src, dst) && !src.is_conj() && !src.is_neg();
    if (!dense_same) {
      // Convert on the host (cheap relative to PCIe) into a staging tensor shaped like dst, then re-enter.
      at::Tensor staged = at::empty(dst.sizes(), src.options().dtype(dst.scalar_type()));
      staged.copy_(src.expand_as(dst));
      if (dst.is_contiguous()) {
        copy_h2d(staged, dst, false);
      } else {
        at::Tensor tmp = at::empty(dst.sizes(), dst.options());
        copy_h2d(staged, tmp, false);
        copy_d2d(tmp, dst, false);
      }
      return;
    }
  }
  size_t nbytes = (size_t)src.numel() * src.dtype().itemsize();
  if (nbytes == 0) return;
  B200_CUDA_CHECK(cudaMemcpyAsync(dst.mutable_data_ptr(), src.const_data_ptr(), nbytes, cudaMemcpyHostToDevice,
                                  stream.stream()));
  bool pinned = host::record_event(src.const_data_ptr(), src.storage().data_ptr().get_context(), stream);
  if (!(non_blocking && (pinned || host::is_pinned(src.const_data_ptr())))) {
    note_implicit_sync("copy_ host->device (pageable or blocking)");
    B200_CUDA_CHECK(cudaStreamSynchronize(stream.stream()));
  }
}

void copy_d2h(const at::Tensor& src, const at::Tensor& dst, bool non_blocking) {
  c10::DeviceIndex sd = src.device().index();
  DeviceSwitch sw(sd);
  Stream stream = get_current_stream(sd);
  bool direct = src.dtype() == dst.dtype() && !src.is_conj() && !src.is_neg() &&
                ((src.is_contiguous() && dst.is_contiguous()) || same_dense_layout(src, dst));
  if (!direct) {
    // Convert/compact on the device, land in a host staging tensor, finish on the host.
    at::Tensor dev_c = src.to(dst.scalar_type()).contiguous();
    if (dev_c.is_conj() || dev_c.is_neg()) dev_c = dev_c.resolve_conj().resolve_neg();
    at::Tensor staged = at::empty(dev_c.sizes(), dst.options().dtype(dst.scalar_type()));
    copy_d2h(dev_c, staged, false);
    dst.copy_(staged.expand_as(dst));
    return;
  }
  size_t nbytes = (size_t)src.numel() * src.dtype().itemsize();
  if (nbytes == 0) return;
  B200_CUDA_CHECK(cudaMemcpyAsync(dst.mutable_data_ptr(), src.const_data_ptr(), nbytes, cudaMemcpyDeviceToHost,
                                  stream.stream()));
  bool pinned = host::record_event(dst.const_data_ptr(), dst.storage().data_ptr().get_context(), stream);
  if (!(non_blocking && (pinned || host::is_pinned(dst.const_data_ptr())))) {
    note_implicit_sync("copy_ device->host");
    B200_CUDA_CHECK(cudaStreamSynchronize(stream.stream()));
  }
}

at::Tensor copy_from_impl(const at::Tensor& self, const at::Tensor& dst, bool non_blocking) {
  if (self.numel() == 0 && dst.numel() == 0) return dst;
  TORCH_CHECK(self.defined() && dst.defined(), "copy_: undefined tensor");
  if (!self.sizes().equals(dst.sizes())) {
    at::Tensor src_e = self.expand_as(dst);
    return copy_from_impl(src_e, dst, non_blocking);
  }
  if (is_dev(self) && is_dev(dst)) {
    copy_d2d(self, dst, non_blocking);
  } else if (is_dev(dst) && self.device().is_cpu()) {
    copy_h2d(self, dst, non_blocking);
  } else if (is_dev(self) && dst.device().is_cpu()) {
    copy_d2h(self, dst, non_blocking);
  } else if (is_dev(self) && dst.device().is_cuda()) {
    // same silicon, different label: a device-to-device copy on our stream
    bridge::AliasScope scope;
    bridge::CudaStreamMirror m(dst.device().index());
    at::Tensor s = scope.to_cuda(self);
    const_cast<at::Tensor&>(dst).copy_(s, non_blocking);
  } else if (is_dev(dst) && self.device().is_cuda()) {
    bridge::AliasScope scope;
    bridge::CudaStreamMirror m(self.device().index());
    scope.to_cuda(dst).copy_(self, non_blocking);
  } else {
    // other accelerators: bounce through the host
    at::Tensor host_t = self.device().is_cpu() ? self : self.cpu();
    if (is_dev(dst)) copy_h2d(host_t, dst, false); else const_cast<at::Tensor&>(dst).copy_(host_t);
  }
  return dst;
}

at::Tensor copy_from_and_resize_impl(const at::Tensor& self, const at::Tensor& dst) {
  if (dst.numel() == 0) at::native::resize_(dst, self.sizes());
  TORCH_CHECK(self.sizes() == dst.sizes(), "_copy_from_and_resize now only support copy with same size!");
  return copy_from_impl(self, dst, false);
}

at::Scalar local_scalar_dense_impl(const at::Tensor& self) {
  TORCH_CHECK(self.numel() == 1, "a Tensor with ", self.numel(), " elements cannot be converted to Scalar");
  at::Tensor h = at::empty({}, self.options().device(at::kCPU));
  copy_d2h(self.reshape({}), h, false);
  return at::_local_scalar_dense(h);
}

void record_stream(at::Tensor& self, c10::Stream s) {
  TORCH_CHECK(s.device_type() == kDeviceType, "record_stream expects a blackwell stream");
  const c10::DataPtr& p = self.storage().data_ptr();
  c10::Storage cs;
  if (bridge::is_wrapped_cuda(p, &cs)) {
    cudaStream_t raw = stream_from_c10(s);
    auto cstream = raw ? c10::cuda::getStreamFromExternal(raw, s.device_index())
                       : c10::cuda::getDefaultCUDAStream(s.device_index());
    c10::cuda::CUDACachingAllocator::recordStream(cs.data_ptr(), cstream);
    return;
  }
  alloc::get()->record_stream(p, s.device_index(), stream_from_c10(s));
}

at::Tensor pin_memory_impl(const at::Tensor& self, std::optional<c10::Device> device) {
  TORCH_CHECK(self.device().is_cpu(), "cannot pin '", self.toString(), "' only dense CPU tensors can be pinned");
  auto* allocator = host::pinned_allocator();
  auto storage = c10::Storage(c10::Storage::use_byte_size_t(),
                              at::detail::computeStorageNbytes(self.sizes(), self.strides(), self.dtype().itemsize()),
                              allocator, false);
  auto out = at::empty({0}, self.options()).set_(storage, 0, self.sizes(), self.strides());
  out.copy_(self);
  return out;
}

bool is_pinned_impl(const at::Tensor& self, std::optional<c10::Device> device) {
  if (!self.device().is_cpu()) return false;
  return host::is_pinned(self.storage().data());
}

}  // namespace

TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("empty.memory_format", TORCH_FN(empty_memory_format));
  m.impl("empty_strided", TORCH_FN(empty_strided));
  m.impl("resize_", TORCH_FN(resize_));
  m.impl("set_.source_Storage", TORCH_FN(set_source_storage));
  m.impl("set_.source_Storage_storage_offset", TORCH_FN(set_storage));
  m.impl("set_.source_Tensor", TORCH_FN(set_source_tensor));
  m.impl("set_", TORCH_FN(set_empty));
  m.impl("as_strided", TORCH_FN(as_strided));
  m.impl("view", TORCH_FN(view));
  m.impl("_reshape_alias", TORCH_FN(reshape_alias));
  m.impl("unfold", TORCH_FN(unfold));
  m.impl("view_as_real", TORCH_FN(view_as_real));
  m.impl("view_as_complex", TORCH_FN(view_as_complex));
  m.impl("_copy_from", TORCH_FN(copy_from_impl));
  m.impl("_copy_from_and_resize", TORCH_FN(copy_from_and_resize_impl));
  m.impl("_local_scalar_dense", TORCH_FN(local_scalar_dense_impl));
  m.impl("record_stream", TORCH_FN(record_stream));
}

// Pinning is dispatched on the *CPU* tensor with the accelerator's key set by the caller.
TORCH_LIBRARY_IMPL(aten, PrivateUse1, m) {
  m.impl("_pin_memory", TORCH_FN(pin_memory_impl));
  m.impl("is_pinned", TORCH_FN(is_pinned_impl));
}

}  // namespace ops
}  // namespace b200
