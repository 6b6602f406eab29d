// ProcessGroupBCCL: the collective backend of the blackwell device ("bccl").
//
// One NCCL communicator per (group, device) carries bootstrap, broadcast, barrier,
// gather/scatter, point-to-point traffic (pipeline parallelism) and -- unless a hot
// path below claims it -- every other collective.  Hot paths (gradient-bucket
// all-reduce with scale/cast, parameter all-gather, gradient reduce-scatter with
// cast, all-to-all dispatch/combine) run as the backend's own sm_100a kernels that
// load and store peer memory directly over NVLink through a per-group
// SymmetricMemory arena.  Every collective is enqueued on a dedicated
// high-priority communication stream, ordered against the caller's stream with
// events, tracked by a watchdog thread (time-outs, asynchronous NCCL errors) and
// logged in a flight-recorder ring buffer.
// Parity: reference torch_musa/csrc/distributed/ProcessGroupMCCL.{h,cpp} (collective(),
// WorkMCCL, watchdog :1758-1943, flight recorder MCCLUtils.h:184-366, Register.cpp:75-209).
#pragma once

#include "core/Device.h"
#include "core/Stream.h"

#include <nccl.h>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>

#include <atomic>
#include <condition_variable>
#include <deque>
#include <list>
#include <memory>
#include <mutex>
#include <thread>
#include <unordered_map>

namespace b200 {
namespace dist {

class SymmetricMemory;

struct FlightRecord {
  uint64_t id = 0, seq = 0;
  std::string op;
  int64_t in_numel = 0, out_numel = 0;
  std::string dtype;
  std::string state;  // scheduled | completed | timed_out | failed
  bool fused = false; // ran on the backend's own P2P kernel
  double created_s = 0, completed_s = 0;
  float duration_ms = -1.f;
  std::string stack;  // C++ backtrace of the caller (BCCL_TRACE_CPP_STACK=1)
};

class FlightRecorder {
 public:
  explicit FlightRecorder(size_t cap = 2048) : cap_(cap) {}
  uint64_t add(FlightRecord r);
  void complete(uint64_t id, const char* state, float duration_ms);
  std::string dump_json() const;
  std::vector<FlightRecord> entries() const;

 private:
  size_t cap_;
  mutable std::mutex mu_;
  std::deque<FlightRecord> ring_;
  uint64_t next_ = 0;
};

class ProcessGroupBCCL;

class WorkBCCL final : public c10d::Work {
 public:
  WorkBCCL(int rank, c10d::OpType op, uint64_t seq, c10::DeviceIndex device, std::chrono::milliseconds timeout,
           bool timing);
  ~WorkBCCL() override = default;

  bool isCompleted() override;
  bool isSuccess() const override;
  bool wait(std::chrono::milliseconds timeout = ::kNoTimeout) override;
  void synchronize() override;
  void blockCurrentStream() override;
  void abort() override;
  std::vector<at::Tensor> result() override { return outputs_; }
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override { return future_; }
  float getDuration() const override;
  uint64_t getSequencenumber() const override { return seq_; }

  bool timed_out() const;
  void set_exception(std::exception_ptr e);

 private:
  friend class ProcessGroupBCCL;
  uint64_t seq_;
  c10::DeviceIndex device_;
  std::chrono::milliseconds timeout_;
  std::chrono::steady_clock::time_point created_;
  Event start_, end_;
  bool timing_;
  bool blocking_wait_ = false;
  std::vector<at::Tensor> outputs_;
  std::vector<at::Tensor> stash_;  // keeps inputs alive until the work retires
  c10::intrusive_ptr<c10::ivalue::Future> future_;
  uint64_t record_id_ = 0;
  std::atomic<bool> aborted_{false};
  bool test_only_ = false;
  bool captured_ = false;  // issued while a graph was being captured: ordering is the graph's, nothing to poll
  // set when the collective ran on a peer-memory kernel: its bounded waits report through this arena's status word
  std::shared_ptr<SymmetricMemory> symm_;
};

class B200_EXPORT ProcessGroupBCCL final : public c10d::Backend {
 public:
  struct Options : c10d::Backend::Options {
    explicit Options(bool high_priority = true)
        : c10d::Backend::Options("bccl"), is_high_priority_stream(high_priority) {}
    bool is_high_priority_stream;
    bool use_fused_collectives = true;   // backend's own P2P kernels for the hot collectives
    int64_t fused_max_bytes = 64ll << 20;  // arena slice size; larger messages are chunked or go to NCCL
    std::string group_name;
  };

  ProcessGroupBCCL(c10::intrusive_ptr<c10d::Store> store, int rank, int size, c10::intrusive_ptr<Options> opts);
  ~ProcessGroupBCCL() override;

  const std::string getBackendName() const override { return "bccl"; }
  c10::intrusive_ptr<c10d::Backend::Options> getBackendOptions() override { return opts_; }
  bool supportsCoalescing() const override { return true; }
  void setTimeout(std::chrono::milliseconds t) override { opts_->timeout = t; }
  void startCoalescing() override;
  c10::intrusive_ptr<c10d::Work> endCoalescing() override;

  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& tensors, const c10d::BroadcastOptions& o) override;
  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors, const c10d::AllreduceOptions& o) override;
  c10::intrusive_ptr<c10d::Work> allreduce_coalesced(std::vector<at::Tensor>& tensors,
                                                     const c10d::AllreduceCoalescedOptions& o) override;
  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& tensors, const c10d::ReduceOptions& o) override;
  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outs, std::vector<at::Tensor>& ins,
                                           const c10d::AllgatherOptions& o) override;
  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& out, at::Tensor& in, const c10d::AllgatherOptions& o) override;
  c10::intrusive_ptr<c10d::Work> allgather_into_tensor_coalesced(std::vector<at::Tensor>& outs,
                                                                 std::vector<at::Tensor>& ins,
                                                                 const c10d::AllgatherOptions& o) override;
  c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>>& outs, std::vector<at::Tensor>& ins,
                                        const c10d::GatherOptions& o) override;
  c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor>& outs, std::vector<std::vector<at::Tensor>>& ins,
                                         const c10d::ScatterOptions& o) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor>& outs,
                                                std::vector<std::vector<at::Tensor>>& ins,
                                                const c10d::ReduceScatterOptions& o) override;
  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor& out, at::Tensor& in,
                                                      const c10d::ReduceScatterOptions& o) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter_tensor_coalesced(std::vector<at::Tensor>& outs,
                                                                 std::vector<at::Tensor>& ins,
                                                                 const c10d::ReduceScatterOptions& o) override;
  c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor& out, at::Tensor& in, std::vector<int64_t>& out_splits,
                                               std::vector<int64_t>& in_splits, const c10d::AllToAllOptions& o) override;
  c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor>& outs, std::vector<at::Tensor>& ins,
                                          const c10d::AllToAllOptions& o) override;
  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& tensors, int dst, int tag) override;
  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& tensors, int src, int tag) override;
  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& o) override;

  void setSequenceNumberForGroup() override {}
  uint64_t getSequenceNumberForGroup() override { return seq_; }
  void waitForPendingWorks() override;
  void enableCollectivesTiming() override { timing_ = true; }
  void eagerConnectSingleDevice(at::Device device) override;
  c10d::ErrorType getError() override { return error_.load(); }
  void abort() override;
  void shutdown() override;

  // backend-specific API (bound to Python)
  std::string dump_flight_recorder() const { return recorder_.dump_json(); }
  std::vector<FlightRecord> flight_records() const { return recorder_.entries(); }
  std::shared_ptr<SymmetricMemory> symmetric_memory(c10::DeviceIndex device);
  int64_t fused_collective_count() const { return fused_count_.load(); }
  void set_fused_collectives(bool on) { opts_->use_fused_collectives = on; }
  std::string nccl_version() const;
  Stream comm_stream(c10::DeviceIndex device);
  // Test hook: a work whose completion event never fires unless `complete` is called (watchdog tests).
  c10::intrusive_ptr<c10d::Work> make_test_work(std::chrono::milliseconds timeout);

 private:
  struct Comm {
    ncclComm_t comm = nullptr;
    Stream stream;
    explicit Comm(Stream s) : stream(s) {}
  };
  Comm& get_comm(c10::DeviceIndex device);
  template <class Fn>
  c10::intrusive_ptr<c10d::Work> collective(c10d::OpType type, const char* name, std::vector<at::Tensor> inputs,
                                            std::vector<at::Tensor> outputs, Fn fn, bool fused = false);
  void enqueue(c10::intrusive_ptr<WorkBCCL> w);
  void watchdog_loop();
  void monitor_loop();   // heartbeat monitor: notices a watchdog thread that stopped making progress
  void check_tensor(const at::Tensor& t, const char* what) const;
  bool try_fused_allreduce(at::Tensor& t, const c10d::ReduceOp& op, cudaStream_t s, c10::DeviceIndex dev);
  bool try_fused_allgather(at::Tensor& out, at::Tensor& in, cudaStream_t s, c10::DeviceIndex dev);
  bool try_fused_alltoall_equal(at::Tensor& out, at::Tensor& in, cudaStream_t s, c10::DeviceIndex dev);
  bool try_fused_reduce_scatter(at::Tensor& out, at::Tensor& in, const c10d::ReduceOp& op, cudaStream_t s,
                                c10::DeviceIndex dev);

  c10::intrusive_ptr<c10d::Store> store_;
  c10::intrusive_ptr<Options> opts_;
  std::mutex mu_;
  std::unordered_map<int, std::unique_ptr<Comm>> comms_;
  std::unordered_map<int, std::shared_ptr<SymmetricMemory>> symm_;
  std::atomic<uint64_t> seq_{0};
  bool timing_ = false;
  bool blocking_wait_ = false;
  int coalescing_ = 0;
  std::vector<at::Tensor> coalesced_tensors_;
  c10::DeviceIndex coalesced_device_ = -1;

  std::thread watchdog_;
  std::thread monitor_;
  std::atomic<uint64_t> heartbeat_{0};
  std::mutex monitor_mu_;
  std::condition_variable monitor_cv_;
  bool monitoring_ = true, propagate_error_ = true, dump_on_timeout_ = false;
  bool trace_stack_ = false, desync_debug_ = false;
  int async_error_handling_ = 1;
  void dump_trace_file();
  void report_desync(uint64_t seq);
  int heartbeat_timeout_s_ = 480;
  std::mutex work_mu_;
  std::condition_variable work_cv_;
  std::list<c10::intrusive_ptr<WorkBCCL>> works_;
  std::atomic<bool> stop_{false};
  // a collective of this group was recorded into a device graph: the communicator library keeps such a
  // communicator alive until every graph that references it is gone, and a blocking destroy would wait for that
  std::atomic<bool> graph_captured_{false};
  std::atomic<c10d::ErrorType> error_{c10d::ErrorType::SUCCESS};
  FlightRecorder recorder_;
  std::atomic<int64_t> fused_count_{0};
};

}  // namespace dist
}  // namespace b200
