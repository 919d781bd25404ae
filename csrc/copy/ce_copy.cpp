#include "ce_copy.h"
#include <chrono>
#include "copy_api.h"

namespace b200ep {

namespace {
using clk = std::chrono::steady_clock;
inline double secs(clk::time_point a, clk::time_point b) {
  return std::chrono::duration<double>(b - a).count();
}
}  // namespace

int ce_can_access_peer(int dev, int peer) {
  int ok = 0;
  if (cudaDeviceCanAccessPeer(&ok, dev, peer) != cudaSuccess) { cudaGetLastError(); return 0; }
  return ok;
}

int ce_enable_peer_access(int dev, int peer) {
  int prev = 0;
  cudaGetDevice(&prev);
  cudaError_t e = cudaSetDevice(dev);
  if (e == cudaSuccess) e = cudaDeviceEnablePeerAccess(peer, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
  cudaSetDevice(prev);
  return (int)e;
}

uint64_t CeEngine::bytes_per_iter() const {
  uint64_t s = 0;
  for (const auto& c : copies_) s += c.nbytes;
  return s;
}

CeEngine::CeEngine(std::vector<CeCopy> copies, int mode, int stream_device, bool use_proxy,
                   int kernel_ctas_per_copy, int kernel_threads)
    : copies_(std::move(copies)), mode_(mode), device_(stream_device), use_proxy_(use_proxy),
      ctas_(kernel_ctas_per_copy), threads_(kernel_threads) {
  int prev = 0;
  cudaGetDevice(&prev);
  cudaSetDevice(device_);
  cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking);
  if (mode_ == kGraph && !copies_.empty()) {
    // Build the graph explicitly: N independent 1-D memcpy nodes (no edges, so the copy
    // engines may run them concurrently); every iteration is then a single graph launch.
    cudaError_t e = cudaGraphCreate(&graph_, 0);
    for (size_t i = 0; e == cudaSuccess && i < copies_.size(); ++i) {
      const auto& c = copies_[i];
      cudaGraphNode_t node;
      e = cudaGraphAddMemcpyNode1D(&node, graph_, nullptr, 0, reinterpret_cast<void*>(c.dst),
                                   reinterpret_cast<const void*>(c.src), c.nbytes, cudaMemcpyDefault);
    }
    if (e == cudaSuccess) e = cudaGraphInstantiate(&graph_exec_, graph_, 0);
    if (e != cudaSuccess) {
      cudaGetLastError();
      graph_exec_ = nullptr;
      last_where_ = std::string("graph build: ") + cudaGetErrorString(e);
    }
  }
  if (mode_ == kKernel && !copies_.empty()) {
    std::vector<CopyDesc> h(copies_.size());
    for (size_t i = 0; i < copies_.size(); ++i) {
      h[i].dst = reinterpret_cast<void*>(copies_[i].dst);
      h[i].src = reinterpret_cast<const void*>(copies_[i].src);
      h[i].nbytes = (long long)copies_[i].nbytes;
    }
    cudaError_t e = cudaMalloc(&desc_dev_, h.size() * sizeof(CopyDesc));
    if (e == cudaSuccess) e = cudaMemcpy(desc_dev_, h.data(), h.size() * sizeof(CopyDesc), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
      // without a valid table the kernel must never be launched: enqueue_once() refuses on a null table
      cudaGetLastError();
      if (desc_dev_) cudaFree(desc_dev_);
      desc_dev_ = nullptr;
      last_where_ = std::string("descriptor table: ") + cudaGetErrorString(e);
    }
  }
  cudaSetDevice(prev);
  if (use_proxy_) proxy_ = std::thread(&CeEngine::proxy_main, this);
}

CeEngine::~CeEngine() {
  if (use_proxy_) {
    { std::lock_guard<std::mutex> l(mu_); stop_ = true; }
    cv_.notify_all();
    if (proxy_.joinable()) proxy_.join();
  }
  if (graph_exec_) cudaGraphExecDestroy(graph_exec_);
  if (graph_) cudaGraphDestroy(graph_);
  if (desc_dev_) cudaFree(desc_dev_);
  if (stream_) cudaStreamDestroy(stream_);
}

int CeEngine::enqueue_once() {
  if (mode_ == kSeparate) {
    for (const auto& c : copies_) {
      cudaError_t e = cudaMemcpyPeerAsync(reinterpret_cast<void*>(c.dst), c.dst_dev,
                                          reinterpret_cast<const void*>(c.src), c.src_dev,
                                          c.nbytes, stream_);
      if (e != cudaSuccess) { last_where_ = "cudaMemcpyPeerAsync"; return (int)e; }
    }
    return 0;
  }
  if (mode_ == kGraph) {
    if (graph_exec_ == nullptr) { if (last_where_.empty()) last_where_ = "graph not instantiated"; return (int)cudaErrorInvalidValue; }
    cudaError_t e = cudaGraphLaunch(graph_exec_, stream_);
    if (e != cudaSuccess) last_where_ = "cudaGraphLaunch";
    return (int)e;
  }
  if (desc_dev_ == nullptr) {
    if (last_where_.empty()) last_where_ = "descriptor table not allocated";
    return (int)cudaErrorInvalidValue;
  }
  if (launch_batched_copy(static_cast<const CopyDesc*>(desc_dev_), (int)copies_.size(), ctas_,
                          threads_, stream_) != 0) {
    last_where_ = "batched copy launch refused";
    return (int)cudaErrorInvalidValue;
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) last_where_ = "batched copy kernel launch";
  return (int)e;
}

// One copy of the list, enqueued by the CALLING thread with no synchronisation: the building
// block of the "one runtime call per copy from the Python thread" comparator
// (`Copy_Engine/nvlink_copy_engine_test.py:551-560` drives its copies that way).
int CeEngine::enqueue_copy(int index) {
  if (index < 0 || index >= (int)copies_.size()) return (int)cudaErrorInvalidValue;
  const CeCopy& c = copies_[index];
  return (int)cudaMemcpyPeerAsync(reinterpret_cast<void*>(c.dst), c.dst_dev,
                                  reinterpret_cast<const void*>(c.src), c.src_dev, c.nbytes, stream_);
}

int CeEngine::synchronize() { return (int)cudaStreamSynchronize(stream_); }

CeResult CeEngine::run_inline(int iters) {
  CeResult r;
  cudaSetDevice(device_);
  const auto t0 = clk::now();
  double submit = 0.0;
  for (int i = 0; i < iters; ++i) {
    const auto a = clk::now();
    const int e = enqueue_once();
    submit += secs(a, clk::now());
    if (e != 0) { r.error = e; r.where = last_where_; break; }
  }
  cudaError_t e = cudaStreamSynchronize(stream_);
  const auto t1 = clk::now();
  if (r.error == 0 && e != cudaSuccess) { r.error = (int)e; r.where = "cudaStreamSynchronize"; }
  r.wall_seconds = secs(t0, t1);
  r.submit_seconds = submit;
  return r;
}

void CeEngine::proxy_main() {
  cudaSetDevice(device_);
  std::unique_lock<std::mutex> l(mu_);
  for (;;) {
    cv_.wait(l, [&] { return has_job_ || stop_; });
    if (stop_) return;
    const int iters = pending_iters_;
    has_job_ = false;
    l.unlock();
    CeResult r = run_inline(iters);
    l.lock();
    job_result_ = r;
    job_done_ = true;
    cv_.notify_all();
  }
}

CeResult CeEngine::run(int iters) {
  if (!use_proxy_) return run_inline(iters);
  std::unique_lock<std::mutex> l(mu_);
  pending_iters_ = iters;
  job_done_ = false;
  has_job_ = true;
  cv_.notify_all();
  cv_.wait(l, [&] { return job_done_; });
  return job_result_;
}

}  // namespace b200ep
