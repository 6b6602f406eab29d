#include "core/Graph.h"

#include "core/Generator.h"

#include <c10/cuda/CUDACachingAllocator.h>

#include <atomic>

namespace b200 {

namespace {
std::atomic<int> g_pending_queries{0};

// Operators of the long tail run on PyTorch's CUDA kernels, which allocate from torch's CUDA caching
// allocator.  While a capture is under way that allocator is pointed at a private pool of its own, keyed
// by the same id in a disjoint id range, so nothing it hands to captured kernels is recycled by eager code.
c10::cuda::MempoolId_t mirror_id(alloc::MempoolId id) {
  return {id.first + 0xB2000000000000ull, id.second + 0xB2000000000000ull};
}
}

bool Graph::is_capturing(cudaStream_t s) {
  cudaStreamCaptureStatus st = cudaStreamCaptureStatusNone;
  B200_CUDA_CHECK(cudaStreamIsCapturing(s, &st));
  return st != cudaStreamCaptureStatusNone;
}

int Graph::pending_event_queries() { return g_pending_queries.load(); }

Graph::~Graph() { reset(); }

void Graph::capture_begin(alloc::MempoolId pool, cudaStreamCaptureMode mode) {
  TORCH_CHECK(!has_exec_ && !capturing_, "This Graph instance already owns a captured graph. To capture a new graph, "
                                         "create a new instance.");
  device_ = current_device();
  Stream stream = get_current_stream(device_);
  TORCH_CHECK(stream.id() != 0, "Graph capture must run on a non-default stream "
                                "(use torch.blackwell.graph(...) or a side stream)");
  capture_stream_ = stream.stream();

  auto* a = alloc::get();
  if (pool.first != 0 || pool.second != 0) {
    pool_ = pool;
    a->create_or_incref_pool(device_, pool_);
  } else {
    pool_ = new_pool_handle();
    a->create_or_incref_pool(device_, pool_);
  }
  pool_owned_ = true;

  // graph-safe RNG state: two int64 words that replay() rewrites before each launch
  seed_dev_ = static_cast<int64_t*>(a->raw_alloc(2 * sizeof(int64_t), device_, capture_stream_));
  offset_dev_ = seed_dev_ + 1;
  auto* gen = at::check_generator<GeneratorImpl>(default_generator(device_));
  {
    std::lock_guard<std::mutex> lock(gen->mutex_);
    gen->capture_prologue(seed_dev_, offset_dev_);
  }

  cudaStream_t cs = capture_stream_;
  a->begin_allocate_to_pool(device_, pool_, [cs](cudaStream_t s) { return s == cs; });
  c10::cuda::CUDACachingAllocator::beginAllocateToPool(device_, mirror_id(pool_), [cs](cudaStream_t s) { return s == cs; });
  capturing_ = true;
  cudaError_t e = cudaStreamBeginCapture(capture_stream_, mode);
  if (e != cudaSuccess) {
    a->end_allocate_to_pool(device_, pool_);
    c10::cuda::CUDACachingAllocator::endAllocateToPool(device_, mirror_id(pool_));
    c10::cuda::CUDACachingAllocator::releasePool(device_, mirror_id(pool_));
    capturing_ = false;
    std::lock_guard<std::mutex> lock(gen->mutex_);
    gen->capture_epilogue();
    B200_CUDA_CHECK(e);
  }
  cudaStreamCaptureStatus st;
  B200_CUDA_CHECK(cudaStreamGetCaptureInfo(capture_stream_, &st, &capture_id_));
  TORCH_INTERNAL_ASSERT(st == cudaStreamCaptureStatusActive);
}

void Graph::capture_end() {
  TORCH_CHECK(capturing_, "capture_end called without a matching capture_begin");
  Stream stream = get_current_stream(device_);
  TORCH_CHECK(stream.stream() == capture_stream_, "Capture must end on the same stream it began on.");
  cudaError_t e = cudaStreamEndCapture(capture_stream_, &graph_);
  alloc::get()->end_allocate_to_pool(device_, pool_);
  c10::cuda::CUDACachingAllocator::endAllocateToPool(device_, mirror_id(pool_));
  cuda_pool_live_ = true;
  capturing_ = false;
  auto* gen = at::check_generator<GeneratorImpl>(default_generator(device_));
  {
    std::lock_guard<std::mutex> lock(gen->mutex_);
    rng_increment_ = gen->capture_epilogue();
  }
  B200_CUDA_CHECK(e);
  TORCH_CHECK(graph_ != nullptr, "Invalid capture.");
  has_graph_ = true;
  B200_CUDA_CHECK(cudaGraphInstantiate(&exec_, graph_, 0));
  has_exec_ = true;
  if (!debug_) {
    B200_CUDA_CHECK(cudaGraphDestroy(graph_));
    has_graph_ = false;
    graph_ = nullptr;
  }
}

void Graph::replay() {
  TORCH_CHECK(has_exec_, "Called Graph::replay without a preceding successful capture.");
  DeviceSwitch sw(device_);
  cudaStream_t s = get_current_stream(device_).stream();
  if (rng_increment_ > 0) {
    auto* gen = at::check_generator<GeneratorImpl>(default_generator(device_));
    int64_t vals[2];
    {
      std::lock_guard<std::mutex> lock(gen->mutex_);
      vals[0] = (int64_t)gen->current_seed();
      vals[1] = (int64_t)gen->get_offset();
      gen->advance_after_replay(rng_increment_);
    }
    // pageable source: the runtime stages the 16 bytes before returning, so the stack buffer may die
    B200_CUDA_CHECK(cudaMemcpyAsync(seed_dev_, vals, sizeof(vals), cudaMemcpyHostToDevice, s));
  }
  B200_CUDA_CHECK(cudaGraphLaunch(exec_, s));
}

void Graph::reinstantiate() {
  TORCH_CHECK(has_graph_, "reinstantiate needs the captured graph: call enable_debug_mode() before capture_begin()");
  if (has_exec_) B200_CUDA_CHECK(cudaGraphExecDestroy(exec_));
  B200_CUDA_CHECK(cudaGraphInstantiate(&exec_, graph_, 0));
  has_exec_ = true;
}

void Graph::reset() {
  if (capturing_) {
    // abandoned capture: end it so the stream is usable again
    cudaGraph_t g = nullptr;
    cudaStreamEndCapture(capture_stream_, &g);
    (void)cudaGetLastError();
    if (g) cudaGraphDestroy(g);
    alloc::get()->end_allocate_to_pool(device_, pool_);
    c10::cuda::CUDACachingAllocator::endAllocateToPool(device_, mirror_id(pool_));
    cuda_pool_live_ = true;
    capturing_ = false;
  }
  if (has_exec_) {
    B200_CUDA_WARN(cudaGraphExecDestroy(exec_));
    has_exec_ = false;
  }
  if (has_graph_) {
    B200_CUDA_WARN(cudaGraphDestroy(graph_));
    has_graph_ = false;
  }
  if (seed_dev_) {
    alloc::get()->raw_delete(seed_dev_);
    seed_dev_ = offset_dev_ = nullptr;
  }
  if (cuda_pool_live_) {
    c10::cuda::CUDACachingAllocator::releasePool(device_, mirror_id(pool_));
    cuda_pool_live_ = false;
  }
  if (pool_owned_) {
    alloc::get()->release_pool(device_, pool_);
    pool_owned_ = false;
  }
}

alloc::MempoolId Graph::pool() const {
  TORCH_CHECK(has_exec_ || capturing_, "Called Graph::pool() without a preceding successful capture.");
  return pool_;
}

void Graph::debug_dump(const std::string& path) {
  TORCH_CHECK(has_graph_, "debug_dump needs enable_debug_mode() before capture_begin()");
  B200_CUDA_CHECK(cudaGraphDebugDotPrint(graph_, path.c_str(), cudaGraphDebugDotFlagsVerbose));
  B200_CUDA_CHECK(cudaGraphDestroy(graph_));
  has_graph_ = false;
}

}  // namespace b200
