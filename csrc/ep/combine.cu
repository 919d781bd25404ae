// Normal-mode combine, standalone form: every received row is pushed back to its source
// rank's combine slot with LSU peer stores, and the source reduces its slots ON ARRIVAL
// (fp32 accumulation, optional per-item weights).
// Replaces `Buffer.combine` as consumed by `DeepEP_v1/deepep_v1_combine.py:241-247` and the
// index_add_ unpermute of `DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:390-403`.
// The fused form (fc2 GEMM epilogue storing tiles straight into the same slots) lives in
// csrc/gemm and uses the reduce role below.
//
// ONE kernel, two roles. A CTA takes a ticket when it starts: the first `n_send` tickets send,
// the rest reduce (so the CTAs that are placed first are senders, whatever order the hardware
// places them in: a sender never waits for anything, a reducer only waits for peers' senders).
//   send role    rows are visited chunk by chunk of the SOURCE's token range (the dispatch
//                told every destination where each source chunk starts in its receive region):
//                all warps work on chunk 0 of every source before chunk 1, a per-segment counter
//                finds the warp that stores a segment's last row, and that warp releases the
//                (destination, chunk) flag on the source.
//   reduce role  tokens in increasing order; before the first token of a chunk the warp waits
//                (bounded) for that chunk's flag from every rank, then sums the token's slots.
// The reduction of chunk c therefore runs while chunk c+1 is still on the wire; only the last
// chunk's reduction is left when the last row arrives.
// With several virtual ranks on one GPU the two roles are launched separately (all sends, then
// all reduces), because a reducer must never be resident while the sender it waits for is not.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "ep.cuh"
#include "api.h"

namespace b200ep {

constexpr int kCombWarps = 16;
constexpr int kCUnroll = 4;

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


// ---- send role ---------------------------------------------------------------------------
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
                                  const PeerPtrs& peers, int si, int n_send, int* s_prefix, int* status) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // slice index: consecutive work items (= neighbouring rows = same peer) land on DIFFERENT CTAs,
  // so every SM stores to a mix of peers and local memory instead of one SM group per peer
  const int gw = warp * n_send + si, nw = n_send * kCombWarps;
  int n = *a.n_recv_ptr;
  if (n > g.cap) n = g.cap;
  if (n < 0) n = 0;

  if (a.bnd == nullptr || g.nch <= 0) {
    // One flag per rank at the end. Rows are grouped by source rank (or by expert), so each warp
    // takes one contiguous slice of the row range: at any instant the running warps cover the
    // whole range, i.e. every peer at once in proportion to its share.
    const int per_warp = (n + nw - 1) / nw;
    const int i_end = min(n, (gw + 1) * per_warp);
    for (int i = gw * per_warp; i < i_end; ++i) combine_copy_row(a, g, rg, peers, i, lane, status);
    if (last_block_arrive(a.block_counter, n_send)) {
      if ((int)threadIdx.x < g.R) {
        int* flag = reinterpret_cast<int*>(peers.base[threadIdx.x] + rg.flags) +
                    kChCombine * kMaxRanks + g.rank;
        st_release_sys(flag, g.epoch);
      }
    }
    return;
  }

  // Segment (c, s) = rows of source s whose token lies in chunk c; visiting order (c, s, row).
  const int R = g.R, nseg = g.nch * R;
  for (int i = threadIdx.x; i < nseg; i += blockDim.x) {
    const int c = i / R, s = i % R;
    int lo = a.bnd[s * kBndStride + c], hi = a.bnd[s * kBndStride + c + 1];
    lo = max(0, min(lo, n));
    hi = max(lo, min(hi, n));
    s_prefix[i] = hi - lo;
  }
  __syncthreads();
  if (si == 0) {
    // a chunk without rows for some source still has to be announced to that source
    for (int i = threadIdx.x; i < nseg; i += blockDim.x) {
      if (s_prefix[i] == 0) {
        int* flag = reinterpret_cast<int*>(peers.base[i % R] + rg.chunk_flags) + g.rank * kMaxCombChunks + i / R;
        st_release_sys(flag, g.epoch);
      }
    }
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    // exclusive scan in place; s_prefix[nseg] = total
    int carry = 0;
    for (int i0 = 0; i0 < nseg; i0 += 32) {
      const int i = i0 + lane;
      const int v = i < nseg ? s_prefix[i] : 0;
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int x = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += x;
      }
      if (i < nseg) s_prefix[i] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) s_prefix[nseg] = carry;
  }
  __syncthreads();
  const int total = s_prefix[nseg];
  for (int i = gw; i < total; i += nw) {
    // last segment whose start is <= i (segments of size 0 share their start with the next one)
    int lo = 0, hi = nseg;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (s_prefix[mid] <= i) lo = mid; else hi = mid;
    }
    const int seg = lo, c = seg / R, s = seg % R;
    const int start = max(0, min(a.bnd[s * kBndStride + c], n));
    combine_copy_row(a, g, rg, peers, start + (i - s_prefix[seg]), lane, status);
    __syncwarp();
    if (lane == 0) {
      // this warp's stores are system-visible before it counts the row; the warp that counts the
      // segment's last row acquires the others' and releases the flag on the source
      fence_acq_rel_sys();
      const int size = s_prefix[seg + 1] - s_prefix[seg];
      const int done = atomicAdd(&a.seg_count[seg], 1) + 1;
      if (done == size) {
        asm volatile("fence.acq_rel.gpu;" ::: "memory");
        a.seg_count[seg] = 0;
        int* flag = reinterpret_cast<int*>(peers.base[s] + rg.chunk_flags) + g.rank * kMaxCombChunks + c;
        st_release_sys(flag, g.epoch);
      }
    }
  }
}

// ---- reduce role -------------------------------------------------------------------------
// warp per token: out[t] = sum_j w[t][j] * comb_x[slot[t][j]]  (w = 1 when absent).
template <typename T>
__device__ void combine_reduce_role(const CombineArgs& a, const EpGeom& g, const EpRegions& rg,
                                    char* self_base, int ri, int n_red, int* status) {
  __shared__ int s_slot[kCombWarps][kMaxItemsPerToken];
  __shared__ float s_w[kCombWarps][kMaxItemsPerToken];
  __shared__ int s_ok;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool by_chunk = a.wait_mode == 2 && g.nch > 0;
  if (a.wait_mode == 1 || (a.wait_mode == 2 && !by_chunk)) {
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
  const char* comb = self_base + rg.comb_x;
  const float* comb_w = reinterpret_cast<const float*>(self_base + rg.comb_w);
  const int* cflags = reinterpret_cast<const int*>(self_base + rg.chunk_flags);
  const int gw = warp * n_red + ri, nw = n_red * kCombWarps;
  int cur_chunk = -1;
  for (int t = gw; t < g.T; t += nw) {
    if (by_chunk) {
      const int c = min(t / g.chunk_tokens, g.nch - 1);
      if (c != cur_chunk) {
        bool ok = true;
        if (lane < g.R)
          ok = wait_flag_ge(cflags + lane * kMaxCombChunks + c, g.epoch, g.timeout_ns, status, kTimeoutCombine);
        if (!__all_sync(0xffffffffu, ok)) return;
        cur_chunk = c;
      }
    }
    int slot = -1;
    if (lane < J) {
      slot = a.send_slot[(size_t)t * J + lane];
      if (slot >= g.slot_cap) slot = -1;
      s_slot[warp][lane] = slot;
      s_w[warp][lane] = a.weights ? a.weights[(size_t)t * J + lane] : 1.f;
    }
    const unsigned vmask = __ballot_sync(0xffffffffu, slot >= 0);
    __syncwarp();
    for (int v = lane; v < nvec; v += 32) {
      float acc[Vec16<T>::N];
#pragma unroll
      for (int q = 0; q < Vec16<T>::N; ++q) acc[q] = 0.f;
      for (unsigned mm = vmask; mm; mm &= mm - 1) {
        const int j = __ffs(mm) - 1;
        const uint4 val = ld_global_v4(comb + (size_t)s_slot[warp][j] * row_bytes + ((size_t)v << 4));
        Vec16<T>::acc(acc, val, s_w[warp][j]);
      }
      st_global_v4(a.out + (size_t)t * row_bytes + ((size_t)v << 4), Vec16<T>::pack(acc));
    }
    if (a.out_topk_w != nullptr) {
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
__global__ void __launch_bounds__(kCombWarps * 32, 2)
combine_kernel(EpGeom g, EpRegions rg, PeerPtrs peers, CombineArgs a, int* status) {
  __shared__ int s_prefix[kMaxRanks * kMaxCombChunks + 1];
  __shared__ unsigned int s_ticket;
  unsigned int tk = blockIdx.x;
  if (a.role == kCombineFused) {
    if (threadIdx.x == 0) {
      const unsigned int got = atomicAdd(a.ticket, 1u);
      if (got == gridDim.x - 1) *a.ticket = 0u;      // every CTA has drawn: ready for the next launch
      s_ticket = got;
    }
    __syncthreads();
    tk = s_ticket;
  }
  const bool sender = a.role == kCombineSendOnly || (a.role == kCombineFused && (int)tk < a.n_send);
  if (sender) {
    combine_send_role(a, g, rg, peers, (int)tk, a.role == kCombineFused ? a.n_send : (int)gridDim.x,
                      s_prefix, status);
  } else {
    const int ri = a.role == kCombineFused ? (int)tk - a.n_send : (int)tk;
    const int n_red = a.role == kCombineFused ? (int)gridDim.x - a.n_send : (int)gridDim.x;
    combine_reduce_role<T>(a, g, rg, peers.base[g.rank], ri, n_red, status);
  }
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
