// See batch_copy_noalloc.h for the contract. The kernel is `batched_copy_kernel` of
// batch_copy.cu (launched through `launch_batched_copy`), reading its descriptor table from
// the static array below instead of from allocated memory.
#include <mutex>
#include "../common.cuh"
#include "batch_copy_noalloc.h"
#include "copy_api.h"

namespace b200ep {

// The scratch: lives in the library image, one instance per GPU that loads it.
static __device__ __align__(256) CopyDesc g_noalloc_table[B200EP_NOALLOC_MAX_COPIES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mu;
CopyDesc* g_table_addr[kMaxDevices] = {};   // device address of g_noalloc_table, per device

// In host code `g_noalloc_table` is only a handle for the symbol, not a device pointer: the
// address that a kernel can use has to be asked for, once per device, with that device current.
int table_for_current_device(CopyDesc** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return -6;
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_table_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_table);
    if (e != cudaSuccess) return (int)e;
    g_table_addr[dev] = static_cast<CopyDesc*>(p);
  }
  *out = g_table_addr[dev];
  return 0;
}
}  // namespace
}  // namespace b200ep

extern "C" int b200ep_batched_copy_noalloc(void* const* dsts, const void* const* srcs, const long long* sizes,
                                           int n, int ctas_per_copy, int threads, cudaStream_t stream) {
  using namespace b200ep;
  if (dsts == nullptr || srcs == nullptr || sizes == nullptr) return -1;
  if (n <= 0) return -2;
  if (n > B200EP_NOALLOC_MAX_COPIES) return -3;
  if (ctas_per_copy <= 0 || ctas_per_copy > 65535 || threads <= 0 || threads > 1024) return -4;
  // The descriptor upload below reads this call's stack. Inside a stream capture it would be
  // recorded as a copy node that keeps the stack address, and every replay would upload whatever
  // then lies there: refuse before anything is issued.
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  cudaError_t ce = cudaStreamIsCapturing(stream, &cap);
  if (ce != cudaSuccess) return (int)ce;
  if (cap != cudaStreamCaptureStatusNone) return -7;
  CopyDesc host[B200EP_NOALLOC_MAX_COPIES];            // on the stack: 24 KiB, no heap
  for (int i = 0; i < n; ++i) {
    if (sizes[i] < 0 || dsts[i] == nullptr || srcs[i] == nullptr) return -5;
    host[i].dst = dsts[i];
    host[i].src = srcs[i];
    host[i].nbytes = sizes[i];
  }
  CopyDesc* table = nullptr;
  const int rc = table_for_current_device(&table);
  if (rc != 0) return rc;
  // Stream-ordered upload: a previous call's kernel on this stream has finished reading the
  // table before these bytes land. The source is pageable stack memory, so the runtime stages it
  // and returns only once it has consumed `host`; the host thread waits for earlier work on the
  // stream while it does so.
  cudaError_t e = cudaMemcpyAsync(table, host, sizeof(CopyDesc) * n, cudaMemcpyHostToDevice, stream);
  if (e != cudaSuccess) return (int)e;
  if (launch_batched_copy(table, n, ctas_per_copy, threads, stream) != 0) return -4;
  e = cudaGetLastError();
  return (int)e;
}

extern "C" const char* b200ep_noalloc_error_string(int code) {
  switch (code) {
    case 0: return "success";
    case -1: return "null pointer array";
    case -2: return "number of copies must be positive";
    case -3: return "too many copies: the static descriptor table holds at most 1024";
    case -4: return "bad launch shape (ctas_per_copy in [1,65535], threads in [1,1024])";
    case -5: return "a copy has a null pointer or a negative size";
    case -6: return "device ordinal outside the supported range";
    case -7: return "not capturable: the stream is being captured and the descriptor upload reads caller stack memory";
    default: return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown error";
  }
}
