#include "distributed/ProcessGroupBCCL.h"

#include <ATen/record_function.h>

#include <cstdio>

#include "aten/Ops.h"
#include "core/Backend.h"
#include "core/CachingAllocator.h"
#include "distributed/SymmetricMemory.h"

#include <ATen/Functions.h>
#include <c10/util/Logging.h>

#include <cstdlib>
#include <sstream>

namespace b200 {
namespace dist {


namespace {

double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

void nccl_check(ncclResult_t r, const char* expr, const char* file, int line) {
  if (r == ncclSuccess || r == ncclInProgress) return;
  TORCH_CHECK_WITH(DistBackendError, false, "bccl: NCCL error in `", expr, "` at ", file, ":", line, ": ",
                   ncclGetErrorString(r), " (", ncclGetLastError(nullptr), ")");
}
#define BCCL_NCCL_CHECK(EXPR) nccl_check((EXPR), #EXPR, __FILE__, __LINE__)

ncclDataType_t nccl_dtype(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return ncclFloat;
    case at::kHalf: return ncclHalf;
    case at::kBFloat16: return ncclBfloat16;
    case at::kDouble: return ncclDouble;
    case at::kInt: return ncclInt32;
    case at::kLong: return ncclInt64;
    case at::kChar: return ncclInt8;
    case at::kByte: return ncclUint8;
    case at::kBool: return ncclUint8;
    case at::kFloat8_e4m3fn: return ncclFloat8e4m3;
    case at::kFloat8_e5m2: return ncclFloat8e5m2;
    default: TORCH_CHECK(false, "bccl: unsupported dtype ", t);
  }
}

ncclRedOp_t nccl_op(const c10d::ReduceOp& op, at::ScalarType t) {
  if (t == at::kBool) {
    // booleans travel as uint8: SUM must not overflow into "false", so it becomes MAX; AVG makes no sense
    TORCH_CHECK(op != c10d::ReduceOp::AVG, "bccl: cannot use ReduceOp.AVG with boolean inputs");
    if (op == c10d::ReduceOp::SUM) return ncclMax;
  }
  switch (op) {
    case c10d::ReduceOp::SUM: return ncclSum;
    case c10d::ReduceOp::AVG: return ncclAvg;
    case c10d::ReduceOp::PRODUCT: return ncclProd;
    case c10d::ReduceOp::MIN: return ncclMin;
    case c10d::ReduceOp::MAX: return ncclMax;
    default: TORCH_CHECK(false, "bccl: unsupported reduce op (BAND/BOR/BXOR/PREMUL_SUM are not available)");
  }
}

// Reduce operator for one NCCL call.  PREMUL_SUM (scale every contribution, then sum: gradient averaging with
// an arbitrary divisor in one pass) needs a per-call custom operator that is destroyed after the enqueue.
struct ReduceOpHolder {
  ncclRedOp_t op;
  ncclComm_t comm = nullptr;
  bool custom = false;
  at::Tensor factor_host;  // keeps the scalar alive until the call is enqueued
  ReduceOpHolder(const c10d::ReduceOp& rop, at::ScalarType t, ncclComm_t c) {
    if (rop == c10d::ReduceOp::PREMUL_SUM) {
      TORCH_CHECK(t == at::kFloat || t == at::kDouble || t == at::kHalf || t == at::kBFloat16,
                  "bccl: PREMUL_SUM needs a floating-point tensor");
      auto* supp = static_cast<const c10d::NCCLPreMulSumSupplement*>(rop.supplement_.get());
      TORCH_CHECK(supp, "bccl: PREMUL_SUM without a factor (use torch.distributed._make_nccl_premul_sum)");
      if (supp->tensor_factor.defined()) {
        const at::Tensor& f = supp->tensor_factor;
        TORCH_CHECK(f.numel() == 1 && f.scalar_type() == t, "bccl: the PREMUL_SUM factor must be one element of the tensor's dtype");
        BCCL_NCCL_CHECK(ncclRedOpCreatePreMulSum(&op, const_cast<void*>(f.const_data_ptr()), nccl_dtype(t),
                                                 f.device().is_cpu() ? ncclScalarHostImmediate : ncclScalarDevice, c));
      } else {
        factor_host = at::scalar_tensor(supp->double_factor, at::TensorOptions().dtype(t).device(at::kCPU));
        BCCL_NCCL_CHECK(ncclRedOpCreatePreMulSum(&op, factor_host.data_ptr(), nccl_dtype(t), ncclScalarHostImmediate, c));
      }
      comm = c;
      custom = true;
    } else {
      op = nccl_op(rop, t);
    }
  }
  ~ReduceOpHolder() {
    if (custom) ncclRedOpDestroy(op, comm);
  }
  ReduceOpHolder(const ReduceOpHolder&) = delete;
  ReduceOpHolder& operator=(const ReduceOpHolder&) = delete;
};

std::string json_escape(const std::string& in) {
  std::string out;
  out.reserve(in.size() + 8);
  for (char ch : in) {
    switch (ch) {
      case '"': out += "\\\""; break;
      case '\\': out += "\\\\"; break;
      case '\n': out += "\\n"; break;
      case '\t': out += "\\t"; break;
      default: if ((unsigned char)ch >= 0x20) out += ch;
    }
  }
  return out;
}

bool capturing(cudaStream_t s);  // defined with the fused-collective helpers below

bool env_flag(const char* name, bool dflt) {
  const char* e = std::getenv(name);
  if (!e) return dflt;
  return std::atoi(e) != 0;
}

at::Tensor flat_real(const at::Tensor& t) { return t.is_complex() ? at::view_as_real(t) : t; }

}  // namespace

// ------------------------------------------------------------------ flight recorder
uint64_t FlightRecorder::add(FlightRecord r) {
  std::lock_guard<std::mutex> g(mu_);
  r.id = next_++;
  r.created_s = now_s();
  if (ring_.size() >= cap_) ring_.pop_front();
  ring_.push_back(std::move(r));
  return ring_.back().id;
}
void FlightRecorder::complete(uint64_t id, const char* state, float duration_ms) {
  std::lock_guard<std::mutex> g(mu_);
  for (auto it = ring_.rbegin(); it != ring_.rend(); ++it) {
    if (it->id == id) {
      it->state = state;
      it->completed_s = now_s();
      it->duration_ms = duration_ms;
      return;
    }
  }
}
std::vector<FlightRecord> FlightRecorder::entries() const {
  std::lock_guard<std::mutex> g(mu_);
  return std::vector<FlightRecord>(ring_.begin(), ring_.end());
}
std::string FlightRecorder::dump_json() const {
  std::ostringstream os;
  os << "{\"version\": 1, \"entries\": [";
  bool first = true;
  for (auto& r : entries()) {
    if (!first) os << ", ";
    first = false;
    os << "{\"id\": " << r.id << ", \"seq\": " << r.seq << ", \"op\": \"" << r.op << "\", \"in_numel\": " << r.in_numel
       << ", \"out_numel\": " << r.out_numel << ", \"dtype\": \"" << r.dtype << "\", \"state\": \"" << r.state
       << "\", \"fused\": " << (r.fused ? "true" : "false") << ", \"created_s\": " << r.created_s
       << ", \"completed_s\": " << r.completed_s << ", \"duration_ms\": " << r.duration_ms;
    if (!r.stack.empty()) os << ", \"stack\": \"" << json_escape(r.stack) << "\"";
    os << "}";
  }
  os << "]}";
  return os.str();
}

// ------------------------------------------------------------------ Work
WorkBCCL::WorkBCCL(int rank, c10d::OpType op, uint64_t seq, c10::DeviceIndex device, std::chrono::milliseconds timeout,
                   bool timing)
    : c10d::Work(rank, op), seq_(seq), device_(device), timeout_(timeout),
      created_(std::chrono::steady_clock::now()), start_(timing ? cudaEventDefault : cudaEventDisableTiming),
      end_(timing ? cudaEventDefault : cudaEventDisableTiming), timing_(timing) {}

bool WorkBCCL::isCompleted() {
  if (aborted_.load() || captured_) return true;
  {
    std::lock_guard<std::mutex> g(mutex_);
    if (exception_) return true;
  }
  return end_.is_created() && end_.query();
}
bool WorkBCCL::isSuccess() const {
  std::lock_guard<std::mutex> g(const_cast<std::mutex&>(mutex_));
  return !exception_;
}
bool WorkBCCL::timed_out() const {
  if (timeout_ == ::kNoTimeout || timeout_.count() <= 0) return false;
  return std::chrono::steady_clock::now() - created_ > timeout_;
}
void WorkBCCL::set_exception(std::exception_ptr e) {
  std::lock_guard<std::mutex> g(mutex_);
  if (!exception_) exception_ = e;
}
void WorkBCCL::blockCurrentStream() {
  if (end_.is_created()) end_.block(get_current_stream(device_));
}
void WorkBCCL::synchronize() { blockCurrentStream(); }
bool WorkBCCL::wait(std::chrono::milliseconds timeout) {
  {
    std::lock_guard<std::mutex> g(mutex_);
    if (exception_) std::rethrow_exception(exception_);
  }
  blockCurrentStream();
  if (captured_) return true;  // the wait above became an edge of the graph; events of a capture cannot be queried
  if (blocking_wait_ || timeout != ::kNoTimeout) {
    // host-side wait with a deadline: poll so a stuck collective turns into an exception, not a hang
    auto limit = timeout != ::kNoTimeout ? timeout : timeout_;
    auto t0 = std::chrono::steady_clock::now();
    while (!isCompleted()) {
      if (limit.count() > 0 && std::chrono::steady_clock::now() - t0 > limit) {
        auto e = std::make_exception_ptr(c10::DistBackendError(
            {__func__, __FILE__, static_cast<uint32_t>(__LINE__)},
            c10::str("bccl: work (seq ", seq_, ") timed out after ", limit.count(), " ms")));
        set_exception(e);
        std::rethrow_exception(e);
      }
      std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
    if (symm_) {
      if (const int st = symm_->peek_status())
        set_exception(std::make_exception_ptr(c10::DistBackendError(
            {__func__, __FILE__, static_cast<uint32_t>(__LINE__)},
            c10::str("bccl: the peer-memory kernel of work seq ", seq_, " gave up waiting for rank ", st - 1))));
    }
    std::lock_guard<std::mutex> g(mutex_);
    if (exception_) std::rethrow_exception(exception_);
  }
  return true;
}
void WorkBCCL::abort() { aborted_ = true; }
float WorkBCCL::getDuration() const {
  TORCH_CHECK(timing_, "bccl: timing is off; call enableCollectivesTiming() or set BCCL_ENABLE_TIMING=1");
  TORCH_CHECK(end_.is_created() && end_.query(), "bccl: work has not finished");
  return start_.elapsed_ms(end_);
}

// ------------------------------------------------------------------ ProcessGroup
ProcessGroupBCCL::ProcessGroupBCCL(c10::intrusive_ptr<c10d::Store> store, int rank, int size,
                                   c10::intrusive_ptr<Options> opts)
    : c10d::Backend(rank, size), store_(std::move(store)), opts_(std::move(opts)),
      recorder_((size_t)(std::getenv("BCCL_TRACE_BUFFER_SIZE") ? std::atoi(std::getenv("BCCL_TRACE_BUFFER_SIZE")) : 2048)) {
  timing_ = env_flag("BCCL_ENABLE_TIMING", false);
  blocking_wait_ = env_flag("BCCL_BLOCKING_WAIT", false);
  if (std::getenv("BCCL_FUSED_COLLECTIVES")) opts_->use_fused_collectives = env_flag("BCCL_FUSED_COLLECTIVES", true);
  if (const char* e = std::getenv("BCCL_SYMM_HALF_MB")) opts_->fused_max_bytes = (int64_t)std::atoll(e) << 20;
  monitoring_ = env_flag("BCCL_ENABLE_MONITORING", true);
  propagate_error_ = env_flag("BCCL_PROPAGATE_ERROR", true);
  dump_on_timeout_ = env_flag("BCCL_DUMP_ON_TIMEOUT", false);
  trace_stack_ = env_flag("BCCL_TRACE_CPP_STACK", false);
  desync_debug_ = env_flag("BCCL_DESYNC_DEBUG", false);
  // 0: a timed-out collective only raises on wait(); 1 (default): the group is also marked failed and the other
  // ranks are told through the store; 2: the communicators are aborted as well so that blocked kernels return
  async_error_handling_ = std::getenv("BCCL_ASYNC_ERROR_HANDLING") ? std::atoi(std::getenv("BCCL_ASYNC_ERROR_HANDLING")) : 1;
  if (const char* e = std::getenv("BCCL_HEARTBEAT_TIMEOUT_SEC")) heartbeat_timeout_s_ = std::max(1, std::atoi(e));
  // device-side waits on other ranks give up after the group's time-out (BCCL_DEVICE_WAIT_MS overrides)
  if (const char* e = std::getenv("BCCL_DEVICE_WAIT_MS")) b200_comm_set_wait_ms(std::atof(e));
  else if (opts_->timeout.count() > 0) b200_comm_set_wait_ms((double)opts_->timeout.count());
  watchdog_ = std::thread([this] { watchdog_loop(); });
  if (monitoring_) monitor_ = std::thread([this] { monitor_loop(); });
}

ProcessGroupBCCL::~ProcessGroupBCCL() {
  stop_ = true;
  work_cv_.notify_all();
  if (watchdog_.joinable()) watchdog_.join();
  monitor_cv_.notify_all();
  if (monitor_.joinable()) monitor_.join();
  std::lock_guard<std::mutex> g(mu_);
  symm_.clear();
  for (auto& kv : comms_) {
    if (kv.second->comm) {
      if (error_.load() == c10d::ErrorType::SUCCESS && !graph_captured_.load()) ncclCommDestroy(kv.second->comm);
      else ncclCommAbort(kv.second->comm);
    }
  }
}

std::string ProcessGroupBCCL::nccl_version() const {
  int v = 0;
  ncclGetVersion(&v);
  return std::to_string(v / 10000) + "." + std::to_string((v / 100) % 100) + "." + std::to_string(v % 100);
}

ProcessGroupBCCL::Comm& ProcessGroupBCCL::get_comm(c10::DeviceIndex device) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = comms_.find(device);
  if (it != comms_.end()) return *it->second;
  DeviceSwitch sw(device);
  auto c = std::make_unique<Comm>(get_stream_from_pool(opts_->is_high_priority_stream, device));
  // rendezvous: rank 0 creates the id and publishes it under a key unique to the device slot.  The store handed to a
  // backend is already prefixed per group, and a process-local counter in the key would differ between members
  // that created their groups in different orders.
  ncclUniqueId id;
  const std::string key = "bccl/uid/" + std::to_string(comms_.size());
  if (rank_ == 0) {
    BCCL_NCCL_CHECK(ncclGetUniqueId(&id));
    store_->set(key, std::vector<uint8_t>(reinterpret_cast<uint8_t*>(&id), reinterpret_cast<uint8_t*>(&id) + sizeof(id)));
  } else {
    auto v = store_->get(key);
    TORCH_CHECK(v.size() == sizeof(id), "bccl: malformed unique id in the store");
    std::memcpy(&id, v.data(), sizeof(id));
  }
  BCCL_NCCL_CHECK(ncclCommInitRank(&c->comm, size_, id, rank_));
  auto& ref = *c;
  comms_.emplace(device, std::move(c));
  return ref;
}

Stream ProcessGroupBCCL::comm_stream(c10::DeviceIndex device) { return get_comm(device).stream; }

void ProcessGroupBCCL::eagerConnectSingleDevice(at::Device device) { get_comm(device.index()); }

std::shared_ptr<SymmetricMemory> ProcessGroupBCCL::symmetric_memory(c10::DeviceIndex device) {
  std::lock_guard<std::mutex> g(mu_);
  auto it = symm_.find(device);
  if (it != symm_.end()) return it->second;
  const std::string key = "bccl/symm/" + std::to_string(symm_.size());
  auto s = std::make_shared<SymmetricMemory>(store_, key, rank_, size_, device, (size_t)opts_->fused_max_bytes);
  if (!s->ok() && rank_ == 0)
    TORCH_WARN("bccl: peer-memory collectives are off for this group (", s->why_not(), "); using NCCL");
  symm_.emplace(device, s);
  return s;
}

void ProcessGroupBCCL::check_tensor(const at::Tensor& t, const char* what) const {
  TORCH_CHECK(t.defined() && t.device().type() == kDeviceType, "bccl ", what, ": expected a blackwell tensor, got ",
              t.defined() ? t.device().str() : "undefined");
  TORCH_CHECK(t.layout() == c10::kStrided && t.is_non_overlapping_and_dense(), "bccl ", what,
              ": tensors must be dense (contiguous in some permutation)");
}

void ProcessGroupBCCL::enqueue(c10::intrusive_ptr<WorkBCCL> w) {
  {
    std::lock_guard<std::mutex> g(work_mu_);
    works_.push_back(std::move(w));
  }
  work_cv_.notify_one();
}

template <class Fn>
c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::collective(c10d::OpType type, const char* name,
                                                            std::vector<at::Tensor> inputs,
                                                            std::vector<at::Tensor> outputs, Fn fn, bool fused) {
  TORCH_CHECK(error_.load() == c10d::ErrorType::SUCCESS,
              "bccl: this process group is in an error state (a previous collective timed out or failed)");
  const at::Tensor& ref = !outputs.empty() ? outputs[0] : inputs[0];
  const c10::DeviceIndex dev = ref.device().index();
  // a profiler range per collective, with the tensors as its inputs (sizes and dtypes show up in traces)
  RECORD_FUNCTION(std::string("bccl:") + name, std::vector<c10::IValue>(inputs.begin(), inputs.end()));
  DeviceSwitch sw(dev);
  Comm& c = get_comm(dev);
  const uint64_t seq = ++seq_;
  auto work = c10::make_intrusive<WorkBCCL>(rank_, type, seq, dev, opts_->timeout, timing_);
  work->blocking_wait_ = blocking_wait_;
  work->outputs_ = outputs;

  FlightRecord rec;
  rec.seq = seq;
  rec.op = name;
  for (auto& t : inputs) rec.in_numel += t.numel();
  for (auto& t : outputs) rec.out_numel += t.numel();
  rec.dtype = c10::toString(ref.scalar_type());
  rec.state = "scheduled";
  rec.fused = fused;
  if (trace_stack_) rec.stack = c10::get_backtrace(/*frames_to_skip=*/2, /*maximum_number_of_frames=*/24);
  work->record_id_ = recorder_.add(std::move(rec));

  // order the communication stream after the producer's stream
  Stream cur = get_current_stream(dev);
  if (coalescing_ == 0 || coalesced_tensors_.empty()) {
    Event ready;
    ready.record(cur);
    ready.block(c.stream);
  }
  if (timing_) work->start_.record(c.stream);
  // the caching allocator must not recycle these blocks before the communication stream is done with them
  auto* a = alloc::get();
  for (auto& t : inputs) a->record_stream(t.storage().data_ptr(), dev, c.stream.stream());
  for (auto& t : outputs) a->record_stream(t.storage().data_ptr(), dev, c.stream.stream());

  const uint64_t fused_before = fused_count_.load();
  try {
    fn(c.comm, c.stream.stream());
  } catch (...) {
    recorder_.complete(work->record_id_, "failed", -1.f);
    error_ = c10d::ErrorType::COMM_ERROR;
    throw;
  }
  if (coalescing_ > 0) {
    for (auto& t : outputs) coalesced_tensors_.push_back(t);
    coalesced_device_ = dev;
    return work;  // the group's single Work is produced by endCoalescing()
  }
  if (fused_count_.load() != fused_before) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = symm_.find(dev);
    if (it != symm_.end()) work->symm_ = it->second;
  }
  work->end_.record(c.stream);
  if (capturing(cur.stream())) {
    // Recorded into a graph: the communication stream forked from the capturing stream at `ready` and joins it
    // again when the caller waits on the work.  The watchdog must not poll events that belong to a capture.
    work->captured_ = true;
    graph_captured_ = true;
    recorder_.complete(work->record_id_, "captured", -1.f);
    return work;
  }
  {
    // future completes on the communication stream
    StreamGuard sg(c.stream);
    std::vector<c10::Device> devices{make_device(dev)};
    work->future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()), devices);
    work->future_->markCompleted(c10::IValue(work->outputs_));
  }
  enqueue(work);
  return work;
}

void ProcessGroupBCCL::startCoalescing() {
  if (coalescing_++ == 0) {
    coalesced_tensors_.clear();
    BCCL_NCCL_CHECK(ncclGroupStart());
  }
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::endCoalescing() {
  TORCH_CHECK(coalescing_ > 0, "bccl: endCoalescing without startCoalescing");
  if (--coalescing_ > 0) return nullptr;
  BCCL_NCCL_CHECK(ncclGroupEnd());
  if (coalesced_device_ < 0) return nullptr;
  const c10::DeviceIndex dev = coalesced_device_;
  coalesced_device_ = -1;
  Comm& c = get_comm(dev);
  auto work = c10::make_intrusive<WorkBCCL>(rank_, c10d::OpType::COALESCED, (uint64_t)seq_, dev, opts_->timeout, timing_);
  work->outputs_ = std::move(coalesced_tensors_);
  coalesced_tensors_.clear();
  FlightRecord rec;
  rec.seq = seq_;
  rec.op = "coalesced";
  rec.state = "scheduled";
  work->record_id_ = recorder_.add(std::move(rec));
  work->end_.record(c.stream);
  {
    StreamGuard sg(c.stream);
    std::vector<c10::Device> devices{make_device(dev)};
    work->future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()), devices);
    work->future_->markCompleted(c10::IValue(work->outputs_));
  }
  enqueue(work);
  return work;
}

// ------------------------------------------------------------------ fused (peer-memory) paths
namespace {
bool fused_dtype(at::ScalarType t) { return t == at::kFloat || t == at::kBFloat16 || t == at::kHalf; }
// The peer-memory kernels take their epoch and arena half as launch arguments, so a replayed graph would reuse
// stale values: while the stream is being captured every rank takes the NCCL path instead (capture state is
// rank-invariant: all ranks capture the same program).
bool capturing(cudaStream_t s) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(s, &st) != cudaSuccess) {
    (void)cudaGetLastError();
    return false;
  }
  return st != cudaStreamCaptureStatusNone;
}
}

bool ProcessGroupBCCL::try_fused_allreduce(at::Tensor& t, const c10d::ReduceOp& op, cudaStream_t s,
                                           c10::DeviceIndex dev) {
  // rank-invariant eligibility only: every rank must take the same branch
  if (!opts_->use_fused_collectives || size_ < 2 || coalescing_ > 0 || capturing(s)) return false;
  if (!(op == c10d::ReduceOp::SUM || op == c10d::ReduceOp::AVG) || !fused_dtype(t.scalar_type())) return false;
  const int64_t n = t.numel();
  const int64_t bytes = n * (int64_t)t.element_size();
  if (n % 8 != 0 || bytes * 2 > opts_->fused_max_bytes || bytes < 1024) return false;
  auto sm = symmetric_memory(dev);
  if (!sm->ok()) return false;
  int64_t half = 0;
  uint32_t epoch = sm->next_epoch(&half);
  const float scale = op == c10d::ReduceOp::AVG ? 1.f / (float)size_ : 1.f;
  const int dt = ops::kdtype(t.scalar_type());
  int e = b200_comm_allreduce(sm->desc(), dt, dt, t.const_data_ptr(), t.mutable_data_ptr(), n, scale, epoch, half,
                              half + ((bytes + 255) / 256) * 256, s);
  TORCH_CHECK(e == 0, "bccl: fused all-reduce launch failed (", cudaGetErrorString((cudaError_t)e),
              "); ranks would diverge, aborting");
  ++fused_count_;
  return true;
}

bool ProcessGroupBCCL::try_fused_allgather(at::Tensor& out, at::Tensor& in, cudaStream_t s, c10::DeviceIndex dev) {
  if (!opts_->use_fused_collectives || size_ < 2 || coalescing_ > 0 || capturing(s)) return false;
  const int64_t bytes = in.numel() * (int64_t)in.element_size();
  if (bytes % 16 != 0 || bytes > opts_->fused_max_bytes || bytes < 1024) return false;
  auto sm = symmetric_memory(dev);
  if (!sm->ok()) return false;
  int64_t half = 0;
  uint32_t epoch = sm->next_epoch(&half);
  int e = b200_comm_allgather(sm->desc(), (int)in.element_size(), in.const_data_ptr(), out.mutable_data_ptr(), bytes,
                              epoch, half, s);
  TORCH_CHECK(e == 0, "bccl: fused all-gather launch failed (", cudaGetErrorString((cudaError_t)e), ")");
  ++fused_count_;
  return true;
}

bool ProcessGroupBCCL::try_fused_reduce_scatter(at::Tensor& out, at::Tensor& in, const c10d::ReduceOp& op,
                                                cudaStream_t s, c10::DeviceIndex dev) {
  if (!opts_->use_fused_collectives || size_ < 2 || coalescing_ > 0 || capturing(s)) return false;
  if (!(op == c10d::ReduceOp::SUM || op == c10d::ReduceOp::AVG) || !fused_dtype(in.scalar_type()) ||
      !fused_dtype(out.scalar_type()))
    return false;
  const int64_t n = out.numel();
  const int64_t in_bytes = in.numel() * (int64_t)in.element_size();
  if (n % 8 != 0 || in_bytes > opts_->fused_max_bytes || in_bytes < 1024) return false;
  if (in.scalar_type() != out.scalar_type() &&
      !((in.scalar_type() == at::kBFloat16 || in.scalar_type() == at::kHalf) && out.scalar_type() == at::kFloat) &&
      !(in.scalar_type() == at::kFloat && out.scalar_type() == at::kBFloat16))
    return false;
  auto sm = symmetric_memory(dev);
  if (!sm->ok()) return false;
  int64_t half = 0;
  uint32_t epoch = sm->next_epoch(&half);
  const float scale = op == c10d::ReduceOp::AVG ? 1.f / (float)size_ : 1.f;
  int e = b200_comm_reduce_scatter(sm->desc(), ops::kdtype(in.scalar_type()), ops::kdtype(out.scalar_type()),
                                   in.const_data_ptr(), out.mutable_data_ptr(), n, scale, epoch, half, s);
  TORCH_CHECK(e == 0, "bccl: fused reduce-scatter launch failed (", cudaGetErrorString((cudaError_t)e), ")");
  ++fused_count_;
  return true;
}

// Equal splits only: every rank can then compute every offset without an exchange of split tables.
bool ProcessGroupBCCL::try_fused_alltoall_equal(at::Tensor& out, at::Tensor& in, cudaStream_t s, c10::DeviceIndex dev) {
  if (!opts_->use_fused_collectives || size_ < 2 || coalescing_ > 0 || capturing(s)) return false;
  const int64_t bytes = in.numel() * (int64_t)in.element_size();
  if (bytes % (16 * size_) != 0 || bytes > opts_->fused_max_bytes || bytes < 1024 || out.numel() != in.numel()) return false;
  auto sm = symmetric_memory(dev);
  if (!sm->ok()) return false;
  const int64_t chunk = bytes / size_;
  std::vector<int64_t> send_off(size_), recv_off(size_), recv_len(size_), peer_send_off(size_);
  for (int r = 0; r < size_; ++r) {
    send_off[r] = r * chunk;
    recv_off[r] = r * chunk;
    recv_len[r] = chunk;
    peer_send_off[r] = rank_ * chunk;
  }
  int64_t half = 0;
  uint32_t epoch = sm->next_epoch(&half);
  int e = b200_comm_alltoall(sm->desc(), in.const_data_ptr(), out.mutable_data_ptr(), bytes, send_off.data(),
                             recv_off.data(), recv_len.data(), peer_send_off.data(), epoch, half, s);
  TORCH_CHECK(e == 0, "bccl: fused all-to-all launch failed (", cudaGetErrorString((cudaError_t)e), ")");
  ++fused_count_;
  return true;
}

// ------------------------------------------------------------------ collectives
c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::broadcast(std::vector<at::Tensor>& tensors,
                                                           const c10d::BroadcastOptions& o) {
  TORCH_CHECK(tensors.size() == 1, "bccl broadcast: expected one tensor");
  check_tensor(tensors[0], "broadcast");
  at::Tensor t = flat_real(tensors[0]);
  const int root = (int)(o.rootRank + o.rootTensor);
  return collective(c10d::OpType::BROADCAST, "broadcast", {t}, {t}, [&](ncclComm_t comm, cudaStream_t s) {
    if (t.numel() == 0) return;
    BCCL_NCCL_CHECK(ncclBroadcast(t.const_data_ptr(), t.mutable_data_ptr(), (size_t)t.numel(), nccl_dtype(t.scalar_type()),
                                  root, comm, s));
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::allreduce(std::vector<at::Tensor>& tensors,
                                                           const c10d::AllreduceOptions& o) {
  TORCH_CHECK(tensors.size() == 1, "bccl allreduce: expected one tensor");
  check_tensor(tensors[0], "allreduce");
  at::Tensor t = tensors[0];
  if (t.is_complex()) {
    TORCH_CHECK(o.reduceOp == c10d::ReduceOp::SUM || o.reduceOp == c10d::ReduceOp::AVG,
                "bccl: complex tensors support only SUM and AVG");
    t = at::view_as_real(t);
  }
  const c10::DeviceIndex dev = t.device().index();
  // decide before scheduling so the flight recorder shows which path ran
  bool fused = false;
  auto w = collective(c10d::OpType::ALLREDUCE, "allreduce", {t}, {tensors[0]}, [&](ncclComm_t comm, cudaStream_t s) {
    if (t.numel() == 0) return;
    if (try_fused_allreduce(t, o.reduceOp, s, dev)) { fused = true; return; }
    ReduceOpHolder rop(o.reduceOp, t.scalar_type(), comm);
    BCCL_NCCL_CHECK(ncclAllReduce(t.const_data_ptr(), t.mutable_data_ptr(), (size_t)t.numel(), nccl_dtype(t.scalar_type()),
                                  rop.op, comm, s));
  });
  (void)fused;
  return w;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::allreduce_coalesced(std::vector<at::Tensor>& tensors,
                                                                     const c10d::AllreduceCoalescedOptions& o) {
  for (auto& t : tensors) check_tensor(t, "allreduce_coalesced");
  return collective(c10d::OpType::ALLREDUCE_COALESCED, "allreduce_coalesced", tensors, tensors,
                    [&](ncclComm_t comm, cudaStream_t s) {
                      BCCL_NCCL_CHECK(ncclGroupStart());
                      for (auto& t : tensors)
                        BCCL_NCCL_CHECK(ncclAllReduce(t.const_data_ptr(), t.mutable_data_ptr(), (size_t)t.numel(),
                                                      nccl_dtype(t.scalar_type()), nccl_op(o.reduceOp, t.scalar_type()),
                                                      comm, s));
                      BCCL_NCCL_CHECK(ncclGroupEnd());
                    });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::reduce(std::vector<at::Tensor>& tensors, const c10d::ReduceOptions& o) {
  TORCH_CHECK(tensors.size() == 1, "bccl reduce: expected one tensor");
  check_tensor(tensors[0], "reduce");
  at::Tensor t = flat_real(tensors[0]);
  const int root = (int)(o.rootRank + o.rootTensor);
  return collective(c10d::OpType::REDUCE, "reduce", {t}, {t}, [&](ncclComm_t comm, cudaStream_t s) {
    BCCL_NCCL_CHECK(ncclReduce(t.const_data_ptr(), t.mutable_data_ptr(), (size_t)t.numel(), nccl_dtype(t.scalar_type()),
                               nccl_op(o.reduceOp, t.scalar_type()), root, comm, s));
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::_allgather_base(at::Tensor& out, at::Tensor& in,
                                                                 const c10d::AllgatherOptions&) {
  check_tensor(out, "all_gather_into_tensor");
  check_tensor(in, "all_gather_into_tensor");
  TORCH_CHECK(out.scalar_type() == in.scalar_type(), "bccl all_gather_into_tensor: dtype mismatch");
  TORCH_CHECK(out.numel() == in.numel() * size_, "bccl all_gather_into_tensor: output must be world_size times the input");
  TORCH_CHECK(out.is_contiguous() && in.is_contiguous(), "bccl all_gather_into_tensor: tensors must be contiguous");
  const c10::DeviceIndex dev = in.device().index();
  return collective(c10d::OpType::_ALLGATHER_BASE, "all_gather_into_tensor", {in}, {out},
                    [&](ncclComm_t comm, cudaStream_t s) {
                      if (in.numel() == 0) return;
                      if (try_fused_allgather(out, in, s, dev)) return;
                      BCCL_NCCL_CHECK(ncclAllGather(in.const_data_ptr(), out.mutable_data_ptr(), (size_t)in.numel(),
                                                    nccl_dtype(in.scalar_type()), comm, s));
                    });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::allgather(std::vector<std::vector<at::Tensor>>& outs,
                                                           std::vector<at::Tensor>& ins, const c10d::AllgatherOptions& o) {
  TORCH_CHECK(ins.size() == 1 && outs.size() == 1 && (int)outs[0].size() == size_,
              "bccl allgather: expected one input and world_size outputs");
  at::Tensor in = ins[0].contiguous();
  check_tensor(in, "allgather");
  bool same = true;
  for (auto& t : outs[0]) same = same && t.sizes() == in.sizes() && t.scalar_type() == in.scalar_type();
  TORCH_CHECK(same, "bccl allgather: all outputs must match the input's shape and dtype");
  // gather into one flat buffer, then scatter views out (device-side copies on the caller's stream after wait)
  at::Tensor flat = at::empty({size_ * in.numel()}, in.options());
  auto w = _allgather_base(flat, in, o);
  w->wait();
  for (int r = 0; r < size_; ++r) outs[0][r].copy_(flat.narrow(0, r * in.numel(), in.numel()).view_as(in));
  return w;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::allgather_into_tensor_coalesced(std::vector<at::Tensor>& outs,
                                                                                 std::vector<at::Tensor>& ins,
                                                                                 const c10d::AllgatherOptions&) {
  TORCH_CHECK(outs.size() == ins.size(), "bccl allgather_into_tensor_coalesced: list size mismatch");
  for (size_t i = 0; i < ins.size(); ++i) { check_tensor(ins[i], "allgather_coalesced"); check_tensor(outs[i], "allgather_coalesced"); }
  return collective(c10d::OpType::COALESCED, "allgather_into_tensor_coalesced", ins, outs,
                    [&](ncclComm_t comm, cudaStream_t s) {
                      BCCL_NCCL_CHECK(ncclGroupStart());
                      for (size_t i = 0; i < ins.size(); ++i)
                        BCCL_NCCL_CHECK(ncclAllGather(ins[i].const_data_ptr(), outs[i].mutable_data_ptr(),
                                                      (size_t)ins[i].numel(), nccl_dtype(ins[i].scalar_type()), comm, s));
                      BCCL_NCCL_CHECK(ncclGroupEnd());
                    });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::_reduce_scatter_base(at::Tensor& out, at::Tensor& in,
                                                                      const c10d::ReduceScatterOptions& o) {
  check_tensor(out, "reduce_scatter_tensor");
  check_tensor(in, "reduce_scatter_tensor");
  TORCH_CHECK(in.numel() == out.numel() * size_, "bccl reduce_scatter_tensor: input must be world_size times the output");
  TORCH_CHECK(out.is_contiguous() && in.is_contiguous(), "bccl reduce_scatter_tensor: tensors must be contiguous");
  const c10::DeviceIndex dev = in.device().index();
  return collective(c10d::OpType::_REDUCE_SCATTER_BASE, "reduce_scatter_tensor", {in}, {out},
                    [&](ncclComm_t comm, cudaStream_t s) {
                      if (out.numel() == 0) return;
                      if (try_fused_reduce_scatter(out, in, o.reduceOp, s, dev)) return;
                      TORCH_CHECK(out.scalar_type() == in.scalar_type(), "bccl reduce_scatter_tensor: dtype mismatch");
                      ReduceOpHolder rop(o.reduceOp, in.scalar_type(), comm);
                      BCCL_NCCL_CHECK(ncclReduceScatter(in.const_data_ptr(), out.mutable_data_ptr(), (size_t)out.numel(),
                                                        nccl_dtype(in.scalar_type()), rop.op, comm, s));
                    });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::reduce_scatter(std::vector<at::Tensor>& outs,
                                                                std::vector<std::vector<at::Tensor>>& ins,
                                                                const c10d::ReduceScatterOptions& o) {
  TORCH_CHECK(outs.size() == 1 && ins.size() == 1 && (int)ins[0].size() == size_,
              "bccl reduce_scatter: expected one output and world_size inputs");
  at::Tensor flat = at::cat(ins[0]).contiguous().view({-1});
  at::Tensor out = outs[0];
  TORCH_CHECK(out.is_contiguous(), "bccl reduce_scatter: output must be contiguous");
  at::Tensor out_flat = out.view({-1});
  return _reduce_scatter_base(out_flat, flat, o);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::reduce_scatter_tensor_coalesced(std::vector<at::Tensor>& outs,
                                                                                 std::vector<at::Tensor>& ins,
                                                                                 const c10d::ReduceScatterOptions& o) {
  TORCH_CHECK(outs.size() == ins.size(), "bccl reduce_scatter_tensor_coalesced: list size mismatch");
  return collective(c10d::OpType::COALESCED, "reduce_scatter_tensor_coalesced", ins, outs,
                    [&](ncclComm_t comm, cudaStream_t s) {
                      BCCL_NCCL_CHECK(ncclGroupStart());
                      for (size_t i = 0; i < ins.size(); ++i)
                        BCCL_NCCL_CHECK(ncclReduceScatter(ins[i].const_data_ptr(), outs[i].mutable_data_ptr(),
                                                          (size_t)outs[i].numel(), nccl_dtype(ins[i].scalar_type()),
                                                          nccl_op(o.reduceOp, ins[i].scalar_type()), comm, s));
                      BCCL_NCCL_CHECK(ncclGroupEnd());
                    });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::alltoall_base(at::Tensor& out, at::Tensor& in,
                                                               std::vector<int64_t>& out_splits,
                                                               std::vector<int64_t>& in_splits,
                                                               const c10d::AllToAllOptions&) {
  check_tensor(out, "all_to_all_single");
  check_tensor(in, "all_to_all_single");
  TORCH_CHECK(out.is_contiguous() && in.is_contiguous(), "bccl all_to_all_single: tensors must be contiguous");
  TORCH_CHECK(out.scalar_type() == in.scalar_type(), "bccl all_to_all_single: dtype mismatch");
  const int64_t row_in = in.dim() > 0 && in.size(0) > 0 ? in.numel() / in.size(0) : 1;
  const int64_t row_out = out.dim() > 0 && out.size(0) > 0 ? out.numel() / out.size(0) : 1;
  std::vector<int64_t> sc(size_), rc(size_), so(size_), ro(size_);
  for (int r = 0; r < size_; ++r) {
    sc[r] = in_splits.empty() ? in.numel() / size_ : in_splits[r] * row_in;
    rc[r] = out_splits.empty() ? out.numel() / size_ : out_splits[r] * row_out;
  }
  int64_t a = 0, b = 0;
  for (int r = 0; r < size_; ++r) { so[r] = a; ro[r] = b; a += sc[r]; b += rc[r]; }
  TORCH_CHECK(a == in.numel() && b == out.numel(), "bccl all_to_all_single: split sizes do not add up");
  const size_t esz = in.element_size();
  const bool equal = in_splits.empty() && out_splits.empty();
  const c10::DeviceIndex dev = in.device().index();
  return collective(c10d::OpType::ALLTOALL_BASE, "all_to_all_single", {in}, {out}, [&, esz](ncclComm_t comm, cudaStream_t s) {
    if (equal && try_fused_alltoall_equal(out, in, s, dev)) return;
    BCCL_NCCL_CHECK(ncclGroupStart());
    for (int r = 0; r < size_; ++r) {
      if (sc[r]) BCCL_NCCL_CHECK(ncclSend(static_cast<const char*>(in.const_data_ptr()) + so[r] * esz, (size_t)sc[r],
                                          nccl_dtype(in.scalar_type()), r, comm, s));
      if (rc[r]) BCCL_NCCL_CHECK(ncclRecv(static_cast<char*>(out.mutable_data_ptr()) + ro[r] * esz, (size_t)rc[r],
                                          nccl_dtype(out.scalar_type()), r, comm, s));
    }
    BCCL_NCCL_CHECK(ncclGroupEnd());
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::alltoall(std::vector<at::Tensor>& outs, std::vector<at::Tensor>& ins,
                                                          const c10d::AllToAllOptions&) {
  TORCH_CHECK((int)outs.size() == size_ && (int)ins.size() == size_, "bccl all_to_all: expected world_size tensors");
  for (auto& t : ins) check_tensor(t, "all_to_all");
  for (auto& t : outs) check_tensor(t, "all_to_all");
  return collective(c10d::OpType::ALLTOALL, "all_to_all", ins, outs, [&](ncclComm_t comm, cudaStream_t s) {
    BCCL_NCCL_CHECK(ncclGroupStart());
    for (int r = 0; r < size_; ++r) {
      if (ins[r].numel())
        BCCL_NCCL_CHECK(ncclSend(ins[r].const_data_ptr(), (size_t)ins[r].numel(), nccl_dtype(ins[r].scalar_type()), r, comm, s));
      if (outs[r].numel())
        BCCL_NCCL_CHECK(ncclRecv(outs[r].mutable_data_ptr(), (size_t)outs[r].numel(), nccl_dtype(outs[r].scalar_type()), r, comm, s));
    }
    BCCL_NCCL_CHECK(ncclGroupEnd());
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::gather(std::vector<std::vector<at::Tensor>>& outs,
                                                        std::vector<at::Tensor>& ins, const c10d::GatherOptions& o) {
  TORCH_CHECK(ins.size() == 1, "bccl gather: expected one input tensor");
  check_tensor(ins[0], "gather");
  const int root = (int)o.rootRank;
  std::vector<at::Tensor> out_list;
  if (rank_ == root) {
    TORCH_CHECK(outs.size() == 1 && (int)outs[0].size() == size_, "bccl gather: root needs world_size outputs");
    out_list = outs[0];
  }
  at::Tensor in = ins[0];
  return collective(c10d::OpType::GATHER, "gather", {in}, out_list, [&, root](ncclComm_t comm, cudaStream_t s) {
    BCCL_NCCL_CHECK(ncclGroupStart());
    if (rank_ == root)
      for (int r = 0; r < size_; ++r)
        BCCL_NCCL_CHECK(ncclRecv(out_list[r].mutable_data_ptr(), (size_t)out_list[r].numel(),
                                 nccl_dtype(out_list[r].scalar_type()), r, comm, s));
    BCCL_NCCL_CHECK(ncclSend(in.const_data_ptr(), (size_t)in.numel(), nccl_dtype(in.scalar_type()), root, comm, s));
    BCCL_NCCL_CHECK(ncclGroupEnd());
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::scatter(std::vector<at::Tensor>& outs,
                                                         std::vector<std::vector<at::Tensor>>& ins,
                                                         const c10d::ScatterOptions& o) {
  TORCH_CHECK(outs.size() == 1, "bccl scatter: expected one output tensor");
  check_tensor(outs[0], "scatter");
  const int root = (int)o.rootRank;
  std::vector<at::Tensor> in_list;
  if (rank_ == root) {
    TORCH_CHECK(ins.size() == 1 && (int)ins[0].size() == size_, "bccl scatter: root needs world_size inputs");
    in_list = ins[0];
  }
  at::Tensor out = outs[0];
  return collective(c10d::OpType::SCATTER, "scatter", in_list, {out}, [&, root](ncclComm_t comm, cudaStream_t s) {
    BCCL_NCCL_CHECK(ncclGroupStart());
    if (rank_ == root)
      for (int r = 0; r < size_; ++r)
        BCCL_NCCL_CHECK(ncclSend(in_list[r].const_data_ptr(), (size_t)in_list[r].numel(),
                                 nccl_dtype(in_list[r].scalar_type()), r, comm, s));
    BCCL_NCCL_CHECK(ncclRecv(out.mutable_data_ptr(), (size_t)out.numel(), nccl_dtype(out.scalar_type()), root, comm, s));
    BCCL_NCCL_CHECK(ncclGroupEnd());
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::send(std::vector<at::Tensor>& tensors, int dst, int) {
  TORCH_CHECK(tensors.size() == 1, "bccl send: expected one tensor");
  check_tensor(tensors[0], "send");
  at::Tensor t = tensors[0];
  return collective(c10d::OpType::SEND, "send", {t}, {}, [&, dst](ncclComm_t comm, cudaStream_t s) {
    BCCL_NCCL_CHECK(ncclSend(t.const_data_ptr(), (size_t)t.numel(), nccl_dtype(t.scalar_type()), dst, comm, s));
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::recv(std::vector<at::Tensor>& tensors, int src, int) {
  TORCH_CHECK(tensors.size() == 1, "bccl recv: expected one tensor");
  check_tensor(tensors[0], "recv");
  at::Tensor t = tensors[0];
  return collective(c10d::OpType::RECV, "recv", {}, {t}, [&, src](ncclComm_t comm, cudaStream_t s) {
    BCCL_NCCL_CHECK(ncclRecv(t.mutable_data_ptr(), (size_t)t.numel(), nccl_dtype(t.scalar_type()), src, comm, s));
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::barrier(const c10d::BarrierOptions& o) {
  c10::DeviceIndex dev = current_device();
  if (o.device.has_value() && o.device->type() == kDeviceType && o.device->has_index()) dev = o.device->index();
  else if (!o.device_ids.empty()) dev = (c10::DeviceIndex)o.device_ids[0];
  DeviceSwitch sw(dev);
  at::Tensor t = at::zeros({8}, at::TensorOptions().dtype(at::kFloat).device(make_device(dev)));
  auto w = collective(c10d::OpType::BARRIER, "barrier", {t}, {t}, [&](ncclComm_t comm, cudaStream_t s) {
    BCCL_NCCL_CHECK(ncclAllReduce(t.const_data_ptr(), t.mutable_data_ptr(), 8, ncclFloat, ncclSum, comm, s));
  });
  // a barrier is a host-level rendezvous: block the host until it is through
  auto* bw = static_cast<WorkBCCL*>(w.get());
  bw->blocking_wait_ = true;
  return w;
}

void ProcessGroupBCCL::waitForPendingWorks() {
  for (;;) {
    {
      std::lock_guard<std::mutex> g(work_mu_);
      if (works_.empty()) return;
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(1));
  }
}

c10::intrusive_ptr<c10d::Work> ProcessGroupBCCL::make_test_work(std::chrono::milliseconds timeout) {
  auto w = c10::make_intrusive<WorkBCCL>(rank_, c10d::OpType::UNKNOWN, ++seq_, (c10::DeviceIndex)0, timeout, false);
  FlightRecord rec;
  rec.seq = w->seq_;
  rec.op = "test_never_completes";
  rec.state = "scheduled";
  w->record_id_ = recorder_.add(std::move(rec));
  w->test_only_ = true;
  enqueue(w);
  return w;
}

// ------------------------------------------------------------------ watchdog
void ProcessGroupBCCL::watchdog_loop() {
  {
    // This thread polls events while other threads may be capturing graphs in the global capture mode, under which
    // an event query from ANY thread invalidates the capture.  Polling is harmless to a capture: opt this thread out.
    cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
    if (cudaThreadExchangeStreamCaptureMode(&mode) != cudaSuccess) (void)cudaGetLastError();
  }
  const auto period = std::chrono::milliseconds(std::getenv("BCCL_WATCHDOG_MS") ? std::atoi(std::getenv("BCCL_WATCHDOG_MS")) : 100);
  while (!stop_.load()) {
    {
      std::unique_lock<std::mutex> lk(work_mu_);
      work_cv_.wait_for(lk, period);
    }
    if (stop_.load()) break;
    const uint64_t beat = heartbeat_.fetch_add(1, std::memory_order_relaxed) + 1;
    // another rank reported a failed collective: surface it here without waiting for our own time-out
    if (propagate_error_ && size_ > 1 && beat % 10 == 0 && error_.load() == c10d::ErrorType::SUCCESS) {
      try {
        const std::string key = std::string("bccl/remote_error");
        if (store_->check({key})) {
          auto v = store_->get(key);
          const std::string who(v.begin(), v.end());
          if (who != std::to_string(rank_)) {
            error_ = c10d::ErrorType::REMOTE_ERROR;
            LOG(ERROR) << "bccl watchdog: rank " << who << " reported a failed collective (seen on rank " << rank_ << ")";
          }
        }
      } catch (...) {
      }
    }
    std::vector<c10::intrusive_ptr<WorkBCCL>> snapshot;
    {
      std::lock_guard<std::mutex> g(work_mu_);
      snapshot.assign(works_.begin(), works_.end());
    }
    for (auto& w : snapshot) {
      bool retire = false;
      try {
        bool done = !w->test_only_ && w->end_.is_created() && w->end_.query();
        const int kst = done && w->symm_ ? w->symm_->peek_status() : 0;
        if (done && kst) {
          // the kernel ran to its end, but only because one of its waits on a peer ran out: its output is not valid
          w->set_exception(std::make_exception_ptr(c10::DistBackendError(
              {__func__, __FILE__, static_cast<uint32_t>(__LINE__)},
              c10::str("bccl: the peer-memory kernel of collective seq ", w->seq_, " on rank ", rank_,
                       " gave up waiting for rank ", kst - 1))));
          recorder_.complete(w->record_id_, "failed", -1.f);
          error_ = c10d::ErrorType::TIMEOUT;
          retire = true;
        } else if (done) {
          float ms = -1.f;
          if (w->timing_) ms = w->start_.elapsed_ms(w->end_);
          recorder_.complete(w->record_id_, "completed", ms);
          retire = true;
        } else if (w->aborted_.load()) {
          recorder_.complete(w->record_id_, "aborted", -1.f);
          retire = true;
        } else if (w->timed_out()) {
          auto e = std::make_exception_ptr(c10::DistBackendError(
              {__func__, __FILE__, static_cast<uint32_t>(__LINE__)},
              c10::str("bccl watchdog: collective seq ", w->seq_, " did not finish within ", w->timeout_.count(),
                       " ms on rank ", rank_)));
          w->set_exception(e);
          recorder_.complete(w->record_id_, "timed_out", -1.f);
          LOG(ERROR) << "bccl watchdog: collective seq " << w->seq_ << " timed out on rank " << rank_
                     << "; flight recorder: " << recorder_.dump_json().substr(0, 2000);
          if (desync_debug_) report_desync(w->seq_);
          if (dump_on_timeout_) dump_trace_file();
          if (async_error_handling_ >= 1) {
            error_ = c10d::ErrorType::TIMEOUT;
            try {
              store_->set(std::string("bccl/remote_error"), std::to_string(rank_));
            } catch (...) {
            }
          }
          if (async_error_handling_ >= 2) {
            std::lock_guard<std::mutex> g(mu_);
            for (auto& kv : comms_)
              if (kv.second->comm) ncclCommAbort(kv.second->comm), kv.second->comm = nullptr;
          }
          retire = true;
        }
      } catch (const std::exception& ex) {
        w->set_exception(std::current_exception());
        recorder_.complete(w->record_id_, "failed", -1.f);
        error_ = c10d::ErrorType::COMM_ERROR;
        retire = true;
      }
      if (retire) {
        std::lock_guard<std::mutex> g(work_mu_);
        works_.remove(w);
      }
    }
    // asynchronous NCCL errors
    {
      std::lock_guard<std::mutex> g(mu_);
      for (auto& kv : comms_) {
        ncclResult_t st = ncclSuccess;
        if (kv.second->comm && ncclCommGetAsyncError(kv.second->comm, &st) == ncclSuccess && st != ncclSuccess &&
            st != ncclInProgress) {
          error_ = c10d::ErrorType::COMM_ERROR;
          LOG(ERROR) << "bccl watchdog: NCCL asynchronous error on rank " << rank_ << ": " << ncclGetErrorString(st);
        }
      }
      for (auto& kv : symm_) {
        if (kv.second && kv.second->ok()) {
          int st = kv.second->take_status();
          if (st) {
            error_ = c10d::ErrorType::TIMEOUT;
            LOG(ERROR) << "bccl watchdog: a peer-memory kernel on rank " << rank_
                       << " gave up waiting for rank " << (st - 1);
          }
        }
      }
    }
  }
}

// Heartbeat monitor: the watchdog bumps a counter every period; if the counter stands still for the heartbeat
// time-out (a watchdog stuck inside a driver or library call), the flight recorder is dumped and the error is
// recorded so that the training loop can react.  The process is never killed from here.
void ProcessGroupBCCL::monitor_loop() {
  uint64_t last = heartbeat_.load();
  auto last_change = std::chrono::steady_clock::now();
  while (!stop_.load()) {
    {
      std::unique_lock<std::mutex> lk(monitor_mu_);
      monitor_cv_.wait_for(lk, std::chrono::seconds(1));
    }
    if (stop_.load()) break;
    const uint64_t now = heartbeat_.load();
    const auto t = std::chrono::steady_clock::now();
    if (now != last) {
      last = now;
      last_change = t;
      continue;
    }
    if (std::chrono::duration_cast<std::chrono::seconds>(t - last_change).count() >= heartbeat_timeout_s_) {
      LOG(ERROR) << "bccl monitor: the watchdog of rank " << rank_ << " made no progress for " << heartbeat_timeout_s_
                 << " s; flight recorder: " << recorder_.dump_json().substr(0, 4000);
      if (dump_on_timeout_) dump_trace_file();
      error_ = c10d::ErrorType::TIMEOUT;
      last_change = t;   // report once per time-out period
    }
  }
}

void ProcessGroupBCCL::dump_trace_file() {
  const char* prefix = std::getenv("BCCL_DEBUG_INFO_TEMP_FILE");
  const std::string path = std::string(prefix ? prefix : "/tmp/bccl_trace_rank_") + std::to_string(rank_);
  if (FILE* f = std::fopen(path.c_str(), "w")) {
    const std::string js = recorder_.dump_json();
    std::fwrite(js.data(), 1, js.size(), f);
    std::fclose(f);
  }
}

// Which collective did every rank reach?  Each rank publishes the sequence number it is stuck on; whoever
// timed out logs the table, which names the rank that fell behind (or never called the collective).
void ProcessGroupBCCL::report_desync(uint64_t seq) {
  try {
    store_->set("bccl/desync/" + std::to_string(rank_), std::to_string(seq));
    std::ostringstream os;
    for (int r = 0; r < size_; ++r) {
      const std::string key = "bccl/desync/" + std::to_string(r);
      if (store_->check({key})) {
        auto v = store_->get(key);
        os << " rank " << r << ": seq " << std::string(v.begin(), v.end()) << ";";
      } else {
        os << " rank " << r << ": no time-out reported;";
      }
    }
    LOG(ERROR) << "bccl desync report from rank " << rank_ << " (stuck at seq " << seq << "):" << os.str();
  } catch (...) {
  }
}

void ProcessGroupBCCL::abort() {
  std::lock_guard<std::mutex> g(mu_);
  for (auto& kv : comms_)
    if (kv.second->comm) {
      ncclCommAbort(kv.second->comm);
      kv.second->comm = nullptr;
    }
  error_ = c10d::ErrorType::COMM_ERROR;
  std::lock_guard<std::mutex> g2(work_mu_);
  for (auto& w : works_) w->abort();
}

void ProcessGroupBCCL::shutdown() {
  waitForPendingWorks();
  std::lock_guard<std::mutex> g(mu_);
  symm_.clear();
  for (auto& kv : comms_)
    if (kv.second->comm) {
      // Graphs that recorded collectives may still be alive (their owner decides when they go): destroying the
      // communicator would block until they are released, so such a communicator is torn down without waiting.
      if (graph_captured_.load()) ncclCommAbort(kv.second->comm);
      else ncclCommDestroy(kv.second->comm);
      kv.second->comm = nullptr;
    }
}

}  // namespace dist
}  // namespace b200
