// CUDA-graph capture and replay for the blackwell device.
//
// capture_begin() routes every allocation made on the capturing stream into a
// private memory pool (so addresses baked into the graph stay valid and are not
// handed to eager code), switches the default generator to its graph-safe mode
// and starts a stream capture; capture_end() instantiates the executable graph;
// replay() refreshes the RNG seed/offset words the captured kernels read and
// launches it.  Parity: reference torch_musa/csrc/aten/musa/MUSAGraph.h:24-92,
// MUSAGraph.cpp:88-244, core/Graph.cpp:10-72.
#pragma once

#include "core/CachingAllocator.h"
#include "core/Device.h"
#include "core/Stream.h"

namespace b200 {

class B200_EXPORT Graph {
 public:
  Graph() = default;
  ~Graph();
  Graph(const Graph&) = delete;
  Graph& operator=(const Graph&) = delete;

  static alloc::MempoolId new_pool_handle() { return alloc::CachingAllocator::new_pool_id(false); }

  void capture_begin(alloc::MempoolId pool = {0, 0}, cudaStreamCaptureMode mode = cudaStreamCaptureModeGlobal);
  void capture_end();
  void replay();
  void reset();
  alloc::MempoolId pool() const;
  void enable_debug_mode() { debug_ = true; }
  void debug_dump(const std::string& path);
  // Re-instantiate the executable graph from the kept cudaGraph_t (needs debug mode or keep_graph).
  void reinstantiate();
  bool has_graph_exec() const { return has_exec_; }

  static bool is_capturing(cudaStream_t s);
  static int pending_event_queries();

 private:
  cudaGraph_t graph_ = nullptr;
  cudaGraphExec_t exec_ = nullptr;
  bool has_graph_ = false, has_exec_ = false, capturing_ = false, debug_ = false;
  alloc::MempoolId pool_{0, 0};
  bool pool_owned_ = false;
  bool cuda_pool_live_ = false;
  c10::DeviceIndex device_ = -1;
  cudaStream_t capture_stream_ = nullptr;
  unsigned long long capture_id_ = 0;
  // graph-safe RNG
  int64_t* seed_dev_ = nullptr;
  int64_t* offset_dev_ = nullptr;
  uint64_t rng_increment_ = 0;
};

}  // namespace b200
