// Normal-mode combine, standalone form: every received row is pushed back to its source
// rank's combine slot with LSU peer stores, and the source reduces its slots "on arrival"
// (fp32 accumulation, optional per-item weights) after a bounded wait on the peers' flags.
// Replaces `Buffer.combine` as consumed by `DeepEP_v1/deepep_v1_combine.py:241-247` and the
// index_add_ unpermute of `DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:390-403`.
// The fused form (fc2 GEMM epilogue storing tiles straight into the same slots) lives in
// csrc/gemm and shares the reduce kernel below.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "ep.cuh"
#include "api.h"

namespace b200ep {

constexpr int kCombWarps = 16;
constexpr int kCUnroll = 4;

__global__ void __launch_bounds__(kCombWarps * 32)
combine_send_kernel(EpGeom g, EpRegions rg, PeerPtrs peers, const int* __restrict__ n_recv_ptr,
                    const int2* __restrict__ recv_meta, const char* __restrict__ x, int row_bytes,
                    const float* __restrict__ topk_w, unsigned int* block_counter, int* status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // slice index: consecutive slices (= neighbouring rows = same peer) land on DIFFERENT CTAs, so
  // every SM stores to a mix of peers and local memory instead of one SM group per peer
  const int gw = warp * gridDim.x + blockIdx.x, nw = gridDim.x * kCombWarps;
  int n = *n_recv_ptr;
  if (n > g.cap) n = g.cap;
  const int nvec = row_bytes >> 4;
  // Rows are grouped by source rank, so consecutive rows go to the SAME peer. Each warp therefore
  // takes one contiguous slice of the row range: at any instant the running warps cover the whole
  // range, i.e. every peer at once in proportion to its share (no incast on one peer at a time).
  const int per_warp = (n + nw - 1) / nw;
  const int i_end = min(n, (gw + 1) * per_warp);
  for (int i = gw * per_warp; i < i_end; ++i) {
    const int2 meta = recv_meta[i];
    const int slot = meta.x, s = meta.y;
    if (s < 0 || s >= g.R || slot < 0 || slot >= g.slot_cap) {
      if (lane == 0) set_status(status, kOverflowSlots);
      continue;
    }
    char* pb = peers.base[s];
    char* dst = pb + rg.comb_x + (size_t)slot * row_bytes;
    const char* src = x + (size_t)i * row_bytes;
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
    if (topk_w != nullptr && lane < wk)
      reinterpret_cast<float*>(pb + rg.comb_w)[(size_t)slot * wk + lane] = topk_w[(size_t)i * wk + lane];
  }
  if (last_block_arrive(block_counter, gridDim.x)) {
    if (threadIdx.x < g.R) {
      int* flag = reinterpret_cast<int*>(peers.base[threadIdx.x] + rg.flags) +
                  kChCombine * kMaxRanks + g.rank;
      st_release_sys(flag, g.epoch);
    }
  }
}

void launch_combine_send(const EpGeom& g, const EpRegions& rg, const PeerPtrs& peers,
                         const int* n_recv_ptr, const int* recv_meta, const char* x, int row_bytes,
                         const float* topk_w, unsigned int* block_counter, int* status, int blocks,
                         cudaStream_t st) {
  if (blocks < 1) blocks = 1;
  combine_send_kernel<<<blocks, kCombWarps * 32, 0, st>>>(
      g, rg, peers, n_recv_ptr, reinterpret_cast<const int2*>(recv_meta), x, row_bytes, topk_w,
      block_counter, status);
}

// Signal only (used when a fused GEMM epilogue has already stored the rows).
__global__ void signal_kernel(PeerPtrs peers, long long flags_off, int channel, int rank, int R,
                              int epoch) {
  if (threadIdx.x < R) {
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

// Reduce: warp per token. out[t] = sum_j w[t][j] * comb_x[slot[t][j]]  (w = 1 when absent).
template <typename T>
__global__ void __launch_bounds__(kCombWarps * 32)
combine_reduce_kernel(EpGeom g, EpRegions rg, char* self_base, const int* __restrict__ send_slot,
                      const float* __restrict__ weights, char* __restrict__ out,
                      float* __restrict__ out_topk_w, int wait_epoch, int* status) {
  __shared__ int s_slot[kCombWarps][kMaxItemsPerToken];
  __shared__ float s_w[kCombWarps][kMaxItemsPerToken];
  __shared__ int ok;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (wait_epoch > 0) {
    if (threadIdx.x == 0) ok = 1;
    __syncthreads();
    if (threadIdx.x < g.R) {
      const int* flags = reinterpret_cast<const int*>(self_base + rg.flags) + kChCombine * kMaxRanks;
      if (!wait_flag_ge(flags + threadIdx.x, wait_epoch, g.timeout_ns, status, kTimeoutCombine)) ok = 0;
    }
    __syncthreads();
    if (!ok) return;
  }
  const int J = g.J;
  const int row_bytes = g.H * (int)sizeof(T);
  const int nvec = row_bytes >> 4;
  const char* comb = self_base + rg.comb_x;
  const float* comb_w = reinterpret_cast<const float*>(self_base + rg.comb_w);
  const int gw = blockIdx.x * kCombWarps + warp, nw = gridDim.x * kCombWarps;
  for (int t = gw; t < g.T; t += nw) {
    int slot = -1;
    if (lane < J) {
      slot = send_slot[(size_t)t * J + lane];
      if (slot >= g.slot_cap) slot = -1;
      s_slot[warp][lane] = slot;
      s_w[warp][lane] = weights ? weights[(size_t)t * J + lane] : 1.f;
    }
    const unsigned vmask = __ballot_sync(0xffffffffu, slot >= 0);
    __syncwarp();
    for (int v = lane; v < nvec; v += 32) {
      float a[Vec16<T>::N];
#pragma unroll
      for (int q = 0; q < Vec16<T>::N; ++q) a[q] = 0.f;
      for (unsigned mm = vmask; mm; mm &= mm - 1) {
        const int j = __ffs(mm) - 1;
        const uint4 val = ld_global_v4(comb + (size_t)s_slot[warp][j] * row_bytes + ((size_t)v << 4));
        Vec16<T>::acc(a, val, s_w[warp][j]);
      }
      st_global_v4(out + (size_t)t * row_bytes + ((size_t)v << 4), Vec16<T>::pack(a));
    }
    if (out_topk_w != nullptr) {
      if (g.mode == 0) {
        // rank mode: [T,K] = sum over destination ranks of the K side values of each row
        if (lane < g.K) {
          float s = 0.f;
          for (unsigned mm = vmask; mm; mm &= mm - 1)
            s += comb_w[(size_t)s_slot[warp][__ffs(mm) - 1] * g.K + lane];
          out_topk_w[(size_t)t * g.K + lane] = s;
        }
      } else if (lane < J) {
        // expert mode: [T,K], entry k is the single side value returned for item (t,k)
        out_topk_w[(size_t)t * J + lane] = slot >= 0 ? comb_w[slot] : 0.f;
      }
    }
    __syncwarp();
  }
}

void launch_combine_reduce(const EpGeom& g, const EpRegions& rg, char* self_base,
                           const int* send_slot, const float* weights, char* out, float* out_topk_w,
                           int dtype_code, int wait_epoch, int* status, int blocks, cudaStream_t st) {
  if (blocks < 1) blocks = 1;
  if (dtype_code == 0)
    combine_reduce_kernel<__nv_bfloat16><<<blocks, kCombWarps * 32, 0, st>>>(
        g, rg, self_base, send_slot, weights, out, out_topk_w, wait_epoch, status);
  else if (dtype_code == 1)
    combine_reduce_kernel<__half><<<blocks, kCombWarps * 32, 0, st>>>(
        g, rg, self_base, send_slot, weights, out, out_topk_w, wait_epoch, status);
  else
    combine_reduce_kernel<float><<<blocks, kCombWarps * 32, 0, st>>>(
        g, rg, self_base, send_slot, weights, out, out_topk_w, wait_epoch, status);
}

}  // namespace b200ep
