#include "aten/CudaAlias.h"

#include "core/Backend.h"
#include "core/Stream.h"

#include <ATen/Context.h>
#include <ATen/core/dispatch/Dispatcher.h>
#include <ATen/cuda/CUDAGeneratorImpl.h>
#include <ATen/detail/CUDAHooksInterface.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAFunctions.h>
#include <torch/library.h>

#include <atomic>
#include <mutex>
#include <unordered_map>

namespace b200 {
namespace bridge {

namespace {

inline bool is_ours(const at::Tensor& t) { return t.defined() && t.device().type() == kDeviceType; }

// DataPtr context that pins another Storage alive.
void storage_ref_deleter(void* ctx) { delete static_cast<c10::Storage*>(ctx); }

std::atomic<int> g_log_level{1};
std::mutex g_count_mu;
std::unordered_map<const c10::FunctionSchema*, int64_t> g_counts;

void note_fallback(const c10::OperatorHandle& op) {
  int lvl = g_log_level.load(std::memory_order_relaxed);
  if (lvl == 0) return;
  bool first;
  {
    std::lock_guard<std::mutex> g(g_count_mu);
    first = (g_counts[&op.schema()]++ == 0);
  }
  if (first && lvl >= 2) {
    TORCH_WARN("blackwell: operator ", toString(op.operator_name()),
               " has no hand-written sm_100a kernel; running PyTorch's CUDA kernel on the same memory");
  }
}

}  // namespace

c10::Storage relabel_storage(const c10::Storage& s, c10::Device dev) {
  auto* keep = new c10::Storage(s);
  c10::DataPtr dp(s.mutable_data(), keep, &storage_ref_deleter, dev);
  c10::Allocator* a = dev.type() == kDeviceType ? c10::GetAllocator(kDeviceType)
                                                : static_cast<c10::Allocator*>(c10::cuda::CUDACachingAllocator::get());
  return c10::Storage(c10::Storage::use_byte_size_t(), s.nbytes(), std::move(dp), a, /*resizable=*/true);
}

c10::Storage wrap_cuda_storage(const c10::Storage& cs) { return relabel_storage(cs, make_device(cs.device().index())); }

bool is_wrapped_cuda(const c10::DataPtr& p, c10::Storage* out) {
  if (p.get_deleter() != &storage_ref_deleter) return false;
  auto* s = static_cast<c10::Storage*>(p.get_context());
  if (!s || s->device().type() != c10::DeviceType::CUDA) return false;
  if (out) *out = *s;
  return true;
}

at::Tensor AliasScope::to_cuda(const at::Tensor& t) {
  if (!is_ours(t)) return t;
  for (auto& e : tensors_)
    if (e.orig.unsafeGetTensorImpl() == t.unsafeGetTensorImpl()) return e.alias;
  TORCH_CHECK(t.layout() == c10::kStrided && !t.is_quantized() && !t.is_nested(),
              "blackwell fallback: only dense strided tensors can be re-labelled as CUDA tensors (got layout ",
              t.layout(), ")");
  c10::StorageImpl* os = t.storage().unsafeGetStorageImpl();
  c10::Storage alias_storage;
  for (auto& sp : storages_)
    if (sp.orig == os) alias_storage = sp.alias;
  if (!alias_storage) {
    c10::Storage wrapped;
    if (is_wrapped_cuda(t.storage().data_ptr(), &wrapped) && wrapped.nbytes() == t.storage().nbytes() &&
        wrapped.data() == t.storage().data()) {
      // This memory came from a CUDA kernel in the first place: hand the original CUDA storage back.
      alias_storage = wrapped;
    } else {
      auto* keep = new c10::Storage(t.storage());
      c10::DataPtr dp(t.storage().mutable_data(), keep, &storage_ref_deleter,
                      c10::Device(c10::DeviceType::CUDA, t.device().index()));
      alias_storage = c10::Storage(c10::Storage::use_byte_size_t(), t.storage().nbytes(), std::move(dp),
                                   c10::cuda::CUDACachingAllocator::get(), /*resizable=*/true);
    }
    storages_.push_back(StoragePair{os, alias_storage, t.storage()});
  }
  auto alias = at::detail::make_tensor<c10::TensorImpl>(c10::Storage(alias_storage),
                                                        c10::DispatchKeySet(c10::DispatchKey::CUDA), t.dtype());
  auto* impl = alias.unsafeGetTensorImpl();
  impl->set_sizes_and_strides(t.sizes(), t.strides(), t.storage_offset());
  if (t.is_conj()) impl->_set_conj(true);
  if (t.is_neg()) impl->_set_neg(true);
  tensors_.push_back(Entry{t, alias, alias_storage.data()});
  return alias;
}

at::Tensor AliasScope::from_cuda(const at::Tensor& t) {
  if (!t.defined() || t.device().type() != c10::DeviceType::CUDA) return t;
  for (auto& e : tensors_)
    if (e.alias.unsafeGetTensorImpl() == t.unsafeGetTensorImpl()) return e.orig;
  c10::StorageImpl* cs = t.storage().unsafeGetStorageImpl();
  c10::Storage target;
  for (auto& sp : storages_)
    if (sp.alias.unsafeGetStorageImpl() == cs) target = sp.orig_storage;
  if (!target) {
    target = wrap_cuda_storage(t.storage());
    storages_.push_back(StoragePair{target.unsafeGetStorageImpl(), t.storage(), target});
  }
  auto out = at::detail::make_tensor<c10::TensorImpl>(std::move(target),
                                                      c10::DispatchKeySet(c10::DispatchKey::PrivateUse1), t.dtype());
  auto* impl = out.unsafeGetTensorImpl();
  impl->set_sizes_and_strides(t.sizes(), t.strides(), t.storage_offset());
  if (t.is_conj()) impl->_set_conj(true);
  if (t.is_neg()) impl->_set_neg(true);
  return out;
}

void AliasScope::sync_back() {
  for (auto& e : tensors_) {
    auto* ai = e.alias.unsafeGetTensorImpl();
    auto* oi = e.orig.unsafeGetTensorImpl();
    const c10::Storage& as = e.alias.storage();
    if (as.data() != e.data_before || as.nbytes() != e.orig.storage().nbytes()) {
      // An out=/in-place kernel reallocated the CUDA view (resize_output): adopt the new memory.
      if (as.data() != e.orig.storage().data()) {
        c10::Storage os = e.orig.storage();
        auto* keep = new c10::Storage(as);
        c10::DataPtr dp(as.mutable_data(), keep, &storage_ref_deleter, make_device(e.orig.device().index()));
        os.unsafeGetStorageImpl()->set_data_ptr_noswap(std::move(dp));
        os.unsafeGetStorageImpl()->set_nbytes(as.nbytes());
      }
      e.data_before = as.data();
    }
    if (ai->sizes() != oi->sizes() || ai->strides() != oi->strides() || ai->storage_offset() != oi->storage_offset()) {
      oi->set_sizes_and_strides(ai->sizes(), ai->strides(), ai->storage_offset());
    }
  }
}

CudaStreamMirror::CudaStreamMirror(c10::DeviceIndex device)
    : prev_(c10::cuda::getCurrentCUDAStream(device)), device_(device) {
  cudaStream_t raw = get_current_stream(device).stream();
  if (raw == nullptr) {
    c10::cuda::setCurrentCUDAStream(c10::cuda::getDefaultCUDAStream(device));
  } else {
    c10::cuda::setCurrentCUDAStream(c10::cuda::getStreamFromExternal(raw, device));
  }
}
CudaStreamMirror::~CudaStreamMirror() { c10::cuda::setCurrentCUDAStream(prev_); }

void cuda_alias_fallback(const c10::OperatorHandle& op, torch::jit::Stack* stack) {
  const auto& schema = op.schema();
  const size_t nargs = schema.arguments().size();
  const size_t base = stack->size() - nargs;
  note_fallback(op);
  lazy_init();
  // PyTorch's CUDA kernels expect its CUDA state (allocator tables, handles) to exist
  static const bool cuda_ready = [] {
    at::globalContext().lazyInitDevice(c10::DeviceType::CUDA);
    return true;
  }();
  (void)cuda_ready;

  AliasScope scope;
  c10::DeviceIndex dev = -1;
  auto see = [&](const at::Tensor& t) {
    if (is_ours(t) && dev < 0) dev = t.device().index();
  };
  for (size_t i = 0; i < nargs; ++i) {
    c10::IValue& iv = (*stack)[base + i];
    if (iv.isTensor()) {
      const at::Tensor& t = iv.toTensor();
      see(t);
      if (is_ours(t)) iv = scope.to_cuda(t);
    } else if (iv.isTensorList()) {
      auto lst = iv.toTensorList();
      c10::List<at::Tensor> out;
      out.reserve(lst.size());
      for (size_t k = 0; k < lst.size(); ++k) {
        at::Tensor t = lst.get(k);
        see(t);
        out.push_back(scope.to_cuda(t));
      }
      iv = std::move(out);
    } else if (iv.isOptionalTensorList()) {
      auto lst = iv.toOptionalTensorList();
      c10::List<std::optional<at::Tensor>> out;
      out.reserve(lst.size());
      for (size_t k = 0; k < lst.size(); ++k) {
        std::optional<at::Tensor> t = lst.get(k);
        if (t.has_value()) {
          see(*t);
          out.push_back(scope.to_cuda(*t));
        } else {
          out.push_back(std::nullopt);
        }
      }
      iv = std::move(out);
    } else if (iv.isDevice()) {
      c10::Device d = iv.toDevice();
      if (d.type() == kDeviceType) {
        c10::DeviceIndex idx = d.has_index() ? d.index() : current_device();
        if (dev < 0) dev = idx;
        iv = c10::Device(c10::DeviceType::CUDA, idx);
      }
    } else if (iv.isGenerator()) {
      at::Generator g = iv.toGenerator();
      if (g.defined() && g.device().type() == kDeviceType) {
        // Random ops of the long tail draw from torch's CUDA generator of the same ordinal; seeding the
        // blackwell device seeds that generator too, so runs stay reproducible.
        iv = at::cuda::detail::getDefaultCUDAGenerator(g.device().index());
      }
    }
  }
  if (dev < 0) dev = current_device();

  {
    DeviceSwitch sw(dev);
    CudaStreamMirror mirror(dev);
    op.callBoxed(stack);
  }
  scope.sync_back();

  const size_t nret = schema.returns().size();
  const size_t rbase = stack->size() - nret;
  for (size_t i = 0; i < nret; ++i) {
    c10::IValue& iv = (*stack)[rbase + i];
    if (iv.isTensor()) {
      iv = scope.from_cuda(iv.toTensor());
    } else if (iv.isTensorList()) {
      auto lst = iv.toTensorList();
      c10::List<at::Tensor> out;
      out.reserve(lst.size());
      for (size_t k = 0; k < lst.size(); ++k) out.push_back(scope.from_cuda(lst.get(k)));
      iv = std::move(out);
    } else if (iv.isOptionalTensorList()) {
      auto lst = iv.toOptionalTensorList();
      c10::List<std::optional<at::Tensor>> out;
      for (size_t k = 0; k < lst.size(); ++k) {
        std::optional<at::Tensor> t = lst.get(k);
        if (t.has_value()) out.push_back(scope.from_cuda(*t)); else out.push_back(std::nullopt);
      }
      iv = std::move(out);
    } else if (iv.isDevice()) {
      c10::Device d = iv.toDevice();
      if (d.type() == c10::DeviceType::CUDA) iv = make_device(d.index());
    }
  }
}

std::vector<std::pair<std::string, int64_t>> fallback_counts() {
  std::lock_guard<std::mutex> g(g_count_mu);
  std::vector<std::pair<std::string, int64_t>> v;
  for (auto& kv : g_counts) v.emplace_back(toString(kv.first->operator_name()), kv.second);
  std::sort(v.begin(), v.end(), [](auto& a, auto& b) { return a.second > b.second; });
  return v;
}
void reset_fallback_counts() {
  std::lock_guard<std::mutex> g(g_count_mu);
  g_counts.clear();
}
void set_fallback_logging(int level) { g_log_level = level; }

namespace {
void boxed(const c10::OperatorHandle& op, torch::jit::Stack* stack) { cuda_alias_fallback(op, stack); }
}  // namespace

TORCH_LIBRARY_IMPL(_, PrivateUse1, m) { m.fallback(torch::CppFunction::makeFromBoxedFunction<&boxed>()); }

}  // namespace bridge
}  // namespace b200
