// Python bindings (the only translation unit that sees torch headers).
// Raw addresses cross the boundary as int64; tensors are checked for device/dtype here.
#include <torch/extension.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <pybind11/stl.h>
#include <chrono>
#include <cstring>
#include <map>

#include "copy/ce_copy.h"
#include "copy/copy_api.h"
#include "ep/api.h"
#include "ep/ll_api.h"
#include "gemm/gemm_api.h"

namespace py = pybind11;
using namespace b200ep;

namespace {

void cuda_ok(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    cudaGetLastError();
    throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
  }
}
cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
template <typename T> T* ptr(int64_t a) { return reinterpret_cast<T*>(static_cast<uintptr_t>(a)); }
template <typename T> T* tptr(const c10::optional<torch::Tensor>& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->is_contiguous(), "expected a contiguous CUDA tensor");
  return reinterpret_cast<T*>(t->data_ptr());
}
template <typename T> T* tptr(const torch::Tensor& t) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous(), "expected a contiguous CUDA tensor");
  return reinterpret_cast<T*>(t.data_ptr());
}

// ---- runtime: symmetric memory over CUDA IPC, pinned mapped words -----------------------
int64_t symm_alloc(int64_t bytes) {
  void* p = nullptr;
  cuda_ok(cudaMalloc(&p, (size_t)bytes), "cudaMalloc(symmetric region)");
  cuda_ok(cudaMemset(p, 0, (size_t)bytes), "cudaMemset(symmetric region)");
  cuda_ok(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  return (int64_t)(uintptr_t)p;
}
void symm_free(int64_t p) { cudaFree(ptr<void>(p)); cudaGetLastError(); }
py::bytes ipc_export(int64_t p) {
  cudaIpcMemHandle_t h;
  cuda_ok(cudaIpcGetMemHandle(&h, ptr<void>(p)), "cudaIpcGetMemHandle");
  return py::bytes(reinterpret_cast<const char*>(&h), sizeof(h));
}
int64_t ipc_open(const std::string& raw) {
  TORCH_CHECK(raw.size() == sizeof(cudaIpcMemHandle_t), "bad IPC handle size");
  cudaIpcMemHandle_t h;
  std::memcpy(&h, raw.data(), sizeof(h));
  void* p = nullptr;
  cuda_ok(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return (int64_t)(uintptr_t)p;
}
void ipc_close(int64_t p) { cudaIpcCloseMemHandle(ptr<void>(p)); cudaGetLastError(); }
int64_t host_mapped_alloc(int64_t bytes) {
  void* p = nullptr;
  cuda_ok(cudaHostAlloc(&p, (size_t)bytes, cudaHostAllocMapped | cudaHostAllocPortable), "cudaHostAlloc");
  std::memset(p, 0, (size_t)bytes);
  return (int64_t)(uintptr_t)p;
}
void host_mapped_free(int64_t p) { cudaFreeHost(ptr<void>(p)); cudaGetLastError(); }
int host_read_i32(int64_t p, int64_t idx) { return reinterpret_cast<volatile int*>(ptr<int>(p))[idx]; }
std::vector<int> host_read_i32_list(int64_t p, int64_t start, int64_t n) {
  volatile int* w = reinterpret_cast<volatile int*>(ptr<int>(p)) + start;
  std::vector<int> out((size_t)n);
  for (int64_t i = 0; i < n; ++i) out[(size_t)i] = w[i];
  return out;
}
void host_write_i32(int64_t p, int64_t idx, int v) { reinterpret_cast<volatile int*>(ptr<int>(p))[idx] = v; }
// Spin on a pinned word until it reaches `want` (GIL released). Returns false on time-out.
bool host_wait_ge(int64_t p, int64_t idx, int want, double timeout_s) {
  py::gil_scoped_release rel;
  volatile int* w = reinterpret_cast<volatile int*>(ptr<int>(p)) + idx;
  const auto t0 = std::chrono::steady_clock::now();
  for (uint64_t it = 0;; ++it) {
    if (*w >= want) return true;
    if ((it & 1023) == 1023 &&
        std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() > timeout_s)
      return false;
  }
}
torch::Tensor view_tensor(int64_t addr, std::vector<int64_t> sizes, const std::string& dtype, int device) {
  static const std::map<std::string, torch::ScalarType> k = {
      {"uint8", torch::kUInt8}, {"int32", torch::kInt32}, {"int64", torch::kInt64},
      {"float32", torch::kFloat32}, {"bfloat16", torch::kBFloat16}, {"float16", torch::kFloat16},
      {"float8_e4m3fn", torch::kFloat8_e4m3fn}, {"bool", torch::kBool}};
  auto it = k.find(dtype);
  TORCH_CHECK(it != k.end(), "unsupported dtype ", dtype);
  return torch::from_blob(ptr<void>(addr), sizes,
                          torch::TensorOptions().dtype(it->second).device(torch::kCUDA, device));
}

PeerPtrs make_peers(const std::vector<int64_t>& bases) {
  TORCH_CHECK((int)bases.size() <= kMaxRanks, "too many ranks");
  PeerPtrs p{};
  for (size_t i = 0; i < bases.size(); ++i) p.base[i] = ptr<char>(bases[i]);
  return p;
}
EpGeom make_geom(const std::vector<int64_t>& v) {
  TORCH_CHECK(v.size() == 16, "geom needs 16 entries");
  EpGeom g{};
  g.rank = (int)v[0]; g.R = (int)v[1]; g.E = (int)v[2]; g.El = (int)v[3]; g.K = (int)v[4];
  g.T = (int)v[5]; g.mode = (int)v[6]; g.J = (int)v[7]; g.B = (int)v[8]; g.H = (int)v[9];
  g.cap = (int)v[10]; g.slot_cap = (int)v[11]; g.epoch = (int)v[12]; g.epoch_wait = (int)v[13];
  g.tail_wait = (int)v[14];
  g.timeout_ns = (unsigned long long)v[15];
  TORCH_CHECK(g.R >= 1 && g.R <= kMaxRanks && g.J <= kMaxItemsPerToken && g.K <= kMaxItemsPerToken,
              "geometry out of range");
  return g;
}
EpRegions make_regions(const std::vector<int64_t>& v) {
  TORCH_CHECK(v.size() == 11, "regions needs 11 entries");
  EpRegions r{};
  r.flags = v[0]; r.counts = v[1]; r.recv_x = v[2]; r.recv_scales = v[3]; r.recv_topk_idx = v[4];
  r.recv_topk_w = v[5]; r.recv_meta = v[6]; r.recv_prob = v[7]; r.comb_x = v[8]; r.comb_w = v[9];
  r.pull_info = v[10];
  return r;
}
// meta tensor layout: [n_recv, send_total, expert_cnt[El], expert_off[El+1], src_off[R+1],
//                      send_base[B], comb_base[B]]
int64_t meta_ints(const EpGeom& g) {
  return 2 + g.El + (g.El + 1) + (g.R + 1) + 2 * (int64_t)g.B;
}
EpMeta make_meta(torch::Tensor& meta, const EpGeom& g) {
  TORCH_CHECK(meta.is_cuda() && meta.scalar_type() == torch::kInt32 && meta.is_contiguous());
  TORCH_CHECK(meta.numel() >= meta_ints(g), "meta tensor too small");
  int* p = meta.data_ptr<int>();
  EpMeta m{};
  m.n_recv = p; m.send_total = p + 1; m.recv_expert_cnt = p + 2;
  m.recv_expert_off = m.recv_expert_cnt + g.El;
  m.recv_src_off = m.recv_expert_off + g.El + 1;
  m.send_base = m.recv_src_off + g.R + 1;
  m.comb_base = m.send_base + g.B;
  return m;
}
void check_launch(const char* what) { cuda_ok(cudaGetLastError(), what); }

}  // namespace

#include "bindings_ep.inc"
#include "bindings_copy.inc"
#include "bindings_ll.inc"
#include "bindings_gemm.inc"

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.attr("MAX_RANKS") = kMaxRanks;
  m.attr("NUM_CHANNELS") = (int)kNumChannels;
  m.attr("CHUNK_TOKENS") = kChunkTokens;
  m.def("counter_reached", [](uint32_t have, uint32_t want) { return counter_reached(have, want); });
  m.def("symm_alloc", &symm_alloc);
  m.def("symm_free", &symm_free);
  m.def("ipc_export", &ipc_export);
  m.def("ipc_open", &ipc_open);
  m.def("ipc_close", &ipc_close);
  m.def("host_mapped_alloc", &host_mapped_alloc);
  m.def("host_mapped_free", &host_mapped_free);
  m.def("host_read_i32", &host_read_i32);
  m.def("host_write_i32", &host_write_i32);
  m.def("host_read_i32_list", &host_read_i32_list);
  m.def("host_wait_ge", &host_wait_ge);
  m.def("view_tensor", &view_tensor);
  bind_ep(m);
  bind_copy(m);
  bind_ll(m);
  bind_gemm(m);
}
