// Normal-mode combine. Replaces `Buffer.combine` as consumed by
// `DeepEP_v1/deepep_v1_combine.py:241-247` and the index_add_ unpermute of
// `DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:390-403`. Two forms:
//
// PULL (rows inside the producer's symmetric region, e.g. the zero-copy output of dispatch):
//   every rank announces where its rows are, waits (bounded) for the peers' announcements and
//   LOADS the rows of its own tokens over NVLink, reducing them in fp32 registers on the way:
//   one pass, no slot region, nothing left to do when the last row has arrived.
// PUSH (rows anywhere): every received row is stored into its slot on the source rank with LSU
//   peer stores; when its own rows are out a CTA waits (bounded) for the peers' flags and reduces
//   the slots of this rank's tokens. The fc2 GEMM epilogue of csrc/gemm stores its tiles into the
//   same slots and is followed by the reduce role alone.
//
// What was measured and dropped: cutting the push into token chunks with one flag per chunk, so
// that the reduction of chunk c overlaps the arrival of chunk c+1. Any release fence on an SM
// whose store queue is full of NVLink stores drains that queue first (tens of microseconds at a
// per-SM share of the link of about 5 GB/s); with 8 ranks the send went from 413 to 587 us with
// one fence per CTA and chunk and to 654 us with the reduction running beside it, against 519 us
// for send-then-reduce. The pull form gets the overlap without any fence.
//
// One CTA of 1024 threads per SM. With several virtual ranks on one GPU the halves that wait for
// peers are launched after the halves they wait for (all announcements / sends first).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "ep.cuh"
#include "api.h"

namespace b200ep {

constexpr int kCombWarps = 32;   // one CTA of 1024 threads per SM
constexpr int kCUnroll = 4;
constexpr int kRUnroll = 4;      // vectors per lane in flight per contributor when reducing

// ---- element helpers -------------------------------------------------------------------
template <typename T> struct Vec16;
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void acc(float* a, const uint4& v, float w) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      a[2 * q] += w * __uint_as_float(u[q] << 16);
      a[2 * q + 1] += w * __uint_as_float(u[q] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* a) {
    uint4 o;
    uint32_t* u = &o.x;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      __nv_bfloat162 h = __floats2bfloat162_rn(a[2 * q], a[2 * q + 1]);
      u[q] = *reinterpret_cast<uint32_t*>(&h);
    }
    return o;
  }
};
template <> struct Vec16<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void acc(float* a, const uint4& v, float w) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const __half2 h = *reinterpret_cast<const __half2*>(&u[q]);
      const float2 f = __half22float2(h);
      a[2 * q] += w * f.x;
      a[2 * q + 1] += w * f.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* a) {
    uint4 o;
    uint32_t* u = &o.x;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      __half2 h = __floats2half2_rn(a[2 * q], a[2 * q + 1]);
      u[q] = *reinterpret_cast<uint32_t*>(&h);
    }
    return o;
  }
};
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void acc(float* a, const uint4& v, float w) {
    a[0] += w * __uint_as_float(v.x);
    a[1] += w * __uint_as_float(v.y);
    a[2] += w * __uint_as_float(v.z);
    a[3] += w * __uint_as_float(v.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* a) {
    return make_uint4(__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]),
                      __float_as_uint(a[3]));
  }
};


// ---- push form: send role ------------------------------------------------------------------
__device__ __forceinline__ void combine_copy_row(const CombineArgs& a, const EpGeom& g, const EpRegions& rg,
                                                 const PeerPtrs& peers, int row, int lane, int* status) {
  const int2 meta = a.recv_meta[row];
  const int slot = meta.x, s = meta.y;
  if (s < 0 || s >= g.R || slot < 0 || slot >= g.slot_cap) {
    if (lane == 0) set_status(status, kOverflowSlots);
    return;
  }
  const int nvec = a.row_bytes >> 4;
  char* pb = peers.base[s];
  char* dst = pb + rg.comb_x + (size_t)slot * a.row_bytes;
  const char* src = a.x + (size_t)row * a.row_bytes;
  for (int v0 = 0; v0 < nvec; v0 += 32 * kCUnroll) {
    uint4 buf[kCUnroll];
#pragma unroll
    for (int u = 0; u < kCUnroll; ++u) {
      const int v = v0 + u * 32 + lane;
      if (v < nvec) buf[u] = ld_global_nc_v4(src + ((size_t)v << 4));
    }
#pragma unroll
    for (int u = 0; u < kCUnroll; ++u) {
      const int v = v0 + u * 32 + lane;
      if (v < nvec) st_global_v4(dst + ((size_t)v << 4), buf[u]);
    }
  }
  // side values returned with the row: K floats per row in rank mode, one in expert mode
  const int wk = g.mode == 0 ? g.K : 1;
  if (a.topk_w != nullptr && lane < wk)
    reinterpret_cast<float*>(pb + rg.comb_w)[(size_t)slot * wk + lane] = a.topk_w[(size_t)row * wk + lane];
}

__device__ void combine_send_role(const CombineArgs& a, const EpGeom& g, const EpRegions& rg,
                                  const PeerPtrs& peers, int* status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  // item index: neighbouring rows (same peer: rows are grouped by source rank or by expert) land on
  // DIFFERENT CTAs, so every SM stores to a mix of peers instead of one SM group per peer; a warp's
  // rows are spread over the whole range, so at any instant all peers are addressed in proportion
  const int gw = warp * gridDim.x + blockIdx.x, nw = gridDim.x * nwarps;
  int n = *a.n_recv_ptr;
  if (n > g.cap) n = g.cap;
  for (int i = gw; i < n; i += nw) combine_copy_row(a, g, rg, peers, i, lane, status);
  if (last_block_arrive(a.block_counter, gridDim.x)) {
    if ((int)threadIdx.x < g.R) {
      int* flag = reinterpret_cast<int*>(peers.base[threadIdx.x] + rg.flags) +
                  kChCombine * kMaxRanks + g.rank;
      st_release_sys(flag, g.epoch);
    }
  }
}

// ---- push form: reduce role ----------------------------------------------------------------
// Work item = (token, part of the row): out[t] = sum_j w[t][j] * comb_x[slot[t][j]]  (w = 1 when absent).
template <typename T>
__device__ void combine_reduce_role(const CombineArgs& a, const EpGeom& g, const EpRegions& rg,
                                    char* self_base, int* status) {
  __shared__ int s_slot[kCombWarps][kMaxItemsPerToken];
  __shared__ float s_w[kCombWarps][kMaxItemsPerToken];
  __shared__ int s_ok;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  if (a.wait) {
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if ((int)threadIdx.x < g.R) {
      const int* flags = reinterpret_cast<const int*>(self_base + rg.flags) + kChCombine * kMaxRanks;
      if (!wait_flag_ge(flags + threadIdx.x, g.epoch, g.timeout_ns, status, kTimeoutCombine)) s_ok = 0;
    }
    __syncthreads();
    if (!s_ok) return;
  }
  const int J = g.J;
  const int row_bytes = g.H * (int)sizeof(T);
  const int nvec = row_bytes >> 4;
  // a row is cut into up to 4 parts of at least 128 vectors, one warp each (shorter dependent chains)
  int parts = nvec / 128;
  parts = parts < 1 ? 1 : (parts > 4 ? 4 : parts);
  if (parts == 3) parts = 2;
  if (nwarps % parts) parts = 1;
  const int part_vec = (nvec + parts - 1) / parts;
  const int tok_per_round = nwarps / parts;
  const int part = warp % parts, tok_in_cta = warp / parts;
  const char* comb = self_base + rg.comb_x;
  const float* comb_w = reinterpret_cast<const float*>(self_base + rg.comb_w);
  const int per_round = gridDim.x * tok_per_round;
  for (int t = blockIdx.x * tok_per_round + tok_in_cta; t < g.T; t += per_round) {
    int slot = -1;
    if (lane < J) {
      slot = a.send_slot[(size_t)t * J + lane];
      if (slot >= g.slot_cap) slot = -1;
      s_slot[warp][lane] = slot;
      s_w[warp][lane] = a.weights ? a.weights[(size_t)t * J + lane] : 1.f;
    }
    const unsigned vmask = __ballot_sync(0xffffffffu, slot >= 0);
    __syncwarp();
    const int v_end = min(nvec, (part + 1) * part_vec);
    // kRUnroll vectors per lane and contributor are loaded together (independent loads in flight),
    // then accumulated in fp32; contributors are visited one after the other.
    for (int v0 = part * part_vec + lane; v0 < v_end; v0 += 32 * kRUnroll) {
      float acc[kRUnroll][Vec16<T>::N];
#pragma unroll
      for (int u = 0; u < kRUnroll; ++u)
#pragma unroll
        for (int q = 0; q < Vec16<T>::N; ++q) acc[u][q] = 0.f;
      for (unsigned mm = vmask; mm; mm &= mm - 1) {
        const int j = __ffs(mm) - 1;
        const char* rowp = comb + (size_t)s_slot[warp][j] * row_bytes;
        const float wj = s_w[warp][j];
        uint4 val[kRUnroll];
#pragma unroll
        for (int u = 0; u < kRUnroll; ++u) {
          const int v = v0 + u * 32;
          if (v < v_end) val[u] = ld_global_v4(rowp + ((size_t)v << 4));
        }
#pragma unroll
        for (int u = 0; u < kRUnroll; ++u)
          if (v0 + u * 32 < v_end) Vec16<T>::acc(acc[u], val[u], wj);
      }
#pragma unroll
      for (int u = 0; u < kRUnroll; ++u) {
        const int v = v0 + u * 32;
        if (v < v_end) st_global_v4(a.out + (size_t)t * row_bytes + ((size_t)v << 4), Vec16<T>::pack(acc[u]));
      }
    }
    if (a.out_topk_w != nullptr && part == 0) {
      if (g.mode == 0) {
        // rank mode: [T,K] = sum over destination ranks of the K side values of each row
        if (lane < g.K) {
          float s = 0.f;
          for (unsigned mm = vmask; mm; mm &= mm - 1)
            s += comb_w[(size_t)s_slot[warp][__ffs(mm) - 1] * g.K + lane];
          a.out_topk_w[(size_t)t * g.K + lane] = s;
        }
      } else if (lane < J) {
        // expert mode: [T,K], entry k is the single side value returned for item (t,k)
        a.out_topk_w[(size_t)t * J + lane] = slot >= 0 ? comb_w[slot] : 0.f;
      }
    }
    __syncwarp();
  }
}

template <typename T>
__global__ void __launch_bounds__(kCombWarps * 32, 1)
combine_kernel(EpGeom g, EpRegions rg, PeerPtrs peers, CombineArgs a, int* status) {
  if (a.role != kCombineReduceOnly) combine_send_role(a, g, rg, peers, status);
  if (a.role != kCombineSendOnly) combine_reduce_role<T>(a, g, rg, peers.base[g.rank], status);
}

int combine_max_ctas() {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 1;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 1) return 1;
  return sms;
}

void launch_combine(const EpGeom& g, const EpRegions& rg, const PeerPtrs& peers, const CombineArgs& a,
                    int dtype_code, int* status, int blocks, cudaStream_t st) {
  if (blocks < 1) blocks = 1;
  if (dtype_code == 0)
    combine_kernel<__nv_bfloat16><<<blocks, kCombWarps * 32, 0, st>>>(g, rg, peers, a, status);
  else if (dtype_code == 1)
    combine_kernel<__half><<<blocks, kCombWarps * 32, 0, st>>>(g, rg, peers, a, status);
  else
    combine_kernel<float><<<blocks, kCombWarps * 32, 0, st>>>(g, rg, peers, a, status);
}

// ---- pull form -----------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kCombWarps * 32, 1)
combine_pull_kernel(EpGeom g, EpRegions rg, PeerPtrs peers, CombinePullArgs a, int* status) {
  __shared__ int s_row[kCombWarps][kMaxItemsPerToken];
  __shared__ int s_src[kCombWarps][kMaxItemsPerToken];
  __shared__ float s_w[kCombWarps][kMaxItemsPerToken];
  __shared__ long long s_info[kMaxRanks][4];
  __shared__ int s_ok;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  char* self_base = peers.base[g.rank];
  if (a.publish && blockIdx.x == 0 && (int)threadIdx.x < g.R) {
    // rows were written by earlier kernels of this stream: complete and visible at this point
    long long* info = reinterpret_cast<long long*>(peers.base[threadIdx.x] + rg.pull_info) + g.rank * 4;
    info[0] = a.x_off;
    info[1] = a.w_off;
    info[2] = a.n_rows;
    int* flag = reinterpret_cast<int*>(peers.base[threadIdx.x] + rg.flags) + kChCombine * kMaxRanks + g.rank;
    st_release_sys(flag, g.epoch);
  }
  if (!a.pull) return;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < g.R) {
    const int* flags = reinterpret_cast<const int*>(self_base + rg.flags) + kChCombine * kMaxRanks;
    if (a.wait && !wait_flag_ge(flags + threadIdx.x, g.epoch, g.timeout_ns, status, kTimeoutCombine)) s_ok = 0;
    const long long* info = reinterpret_cast<const long long*>(self_base + rg.pull_info) + threadIdx.x * 4;
    for (int q = 0; q < 3; ++q) s_info[threadIdx.x][q] = __ldcg(&info[q]);
  }
  __syncthreads();
  if (!s_ok) return;
  const int J = g.J;
  const int row_bytes = g.H * (int)sizeof(T);
  const int nvec = row_bytes >> 4;
  int parts = nvec / 128;
  parts = parts < 1 ? 1 : (parts > 4 ? 4 : parts);
  if (parts == 3) parts = 2;
  if (nwarps % parts) parts = 1;
  const int part_vec = (nvec + parts - 1) / parts;
  const int tok_per_round = nwarps / parts;
  const int part = warp % parts, tok_in_cta = warp / parts;
  // consecutive (token, part) items land on different CTAs: every SM reads from a mix of peers
  const int per_round = gridDim.x * tok_per_round;
  for (int t = tok_in_cta * gridDim.x + blockIdx.x; t < g.T; t += per_round) {
    int row = -1;
    if (lane < J) {
      row = a.send_row[(size_t)t * J + lane];
      int d = lane;
      if (g.mode == 1) {
        const long long e = a.topk_idx[(size_t)t * g.K + lane];
        d = (e >= 0 && e < g.E) ? (int)(e / g.El) : -1;
      }
      if (row >= 0 && (d < 0 || (long long)row >= s_info[d][2] || s_info[d][0] < 0)) {
        set_status(status, kOverflowSlots);       // the peer did not announce that many rows
        row = -1;
      }
      s_row[warp][lane] = row;
      s_src[warp][lane] = d;
      s_w[warp][lane] = a.weights ? a.weights[(size_t)t * J + lane] : 1.f;
    }
    const unsigned vmask = __ballot_sync(0xffffffffu, row >= 0);
    __syncwarp();
    const int v_end = min(nvec, (part + 1) * part_vec);
    for (int v0 = part * part_vec + lane; v0 < v_end; v0 += 32 * kRUnroll) {
      float acc[kRUnroll][Vec16<T>::N];
#pragma unroll
      for (int u = 0; u < kRUnroll; ++u)
#pragma unroll
        for (int q = 0; q < Vec16<T>::N; ++q) acc[u][q] = 0.f;
      for (unsigned mm = vmask; mm; mm &= mm - 1) {
        const int j = __ffs(mm) - 1;
        const int d = s_src[warp][j];
        const char* rowp = peers.base[d] + s_info[d][0] + (size_t)s_row[warp][j] * row_bytes;
        const float wj = s_w[warp][j];
        uint4 val[kRUnroll];
#pragma unroll
        for (int u = 0; u < kRUnroll; ++u) {
          const int v = v0 + u * 32;
          if (v < v_end) val[u] = ld_global_v4(rowp + ((size_t)v << 4));   // coherent path: another GPU wrote these rows
        }
#pragma unroll
        for (int u = 0; u < kRUnroll; ++u)
          if (v0 + u * 32 < v_end) Vec16<T>::acc(acc[u], val[u], wj);
      }
#pragma unroll
      for (int u = 0; u < kRUnroll; ++u) {
        const int v = v0 + u * 32;
        if (v < v_end) st_global_v4(a.out + (size_t)t * row_bytes + ((size_t)v << 4), Vec16<T>::pack(acc[u]));
      }
    }
    if (a.out_topk_w != nullptr && part == 0) {
      // side values: K floats per row in rank mode (summed over the destinations), one in expert mode
      if (g.mode == 0) {
        if (lane < g.K) {
          float s = 0.f;
          for (unsigned mm = vmask; mm; mm &= mm - 1) {
            const int j = __ffs(mm) - 1, d = s_src[warp][j];
            const float* wp = reinterpret_cast<const float*>(peers.base[d] + s_info[d][1]);
            s += wp[(size_t)s_row[warp][j] * g.K + lane];
          }
          a.out_topk_w[(size_t)t * g.K + lane] = s;
        }
      } else if (lane < J) {
        float v = 0.f;
        if (row >= 0) {
          const int d = s_src[warp][lane];
          v = reinterpret_cast<const float*>(peers.base[d] + s_info[d][1])[row];
        }
        a.out_topk_w[(size_t)t * J + lane] = v;
      }
    }
    __syncwarp();
  }
}

void launch_combine_pull(const EpGeom& g, const EpRegions& rg, const PeerPtrs& peers,
                         const CombinePullArgs& a, int dtype_code, int* status, int blocks, cudaStream_t st) {
  if (blocks < 1) blocks = 1;
  const int threads = a.pull ? kCombWarps * 32 : 32;
  if (!a.pull) blocks = 1;
  if (dtype_code == 0)
    combine_pull_kernel<__nv_bfloat16><<<blocks, threads, 0, st>>>(g, rg, peers, a, status);
  else if (dtype_code == 1)
    combine_pull_kernel<__half><<<blocks, threads, 0, st>>>(g, rg, peers, a, status);
  else
    combine_pull_kernel<float><<<blocks, threads, 0, st>>>(g, rg, peers, a, status);
}

// Signal only (used when a fused GEMM epilogue has already stored the rows).
__global__ void signal_kernel(PeerPtrs peers, long long flags_off, int channel, int rank, int R,
                              int epoch) {
  if ((int)threadIdx.x < R) {
    fence_acq_rel_sys();
    int* flag = reinterpret_cast<int*>(peers.base[threadIdx.x] + flags_off) +
                channel * kMaxRanks + rank;
    st_release_sys(flag, epoch);
  }
}
void launch_signal(const PeerPtrs& peers, long long flags_off, int channel, int rank, int R,
                   int epoch, cudaStream_t st) {
  signal_kernel<<<1, 32, 0, st>>>(peers, flags_off, channel, rank, R, epoch);
}

}  // namespace b200ep
