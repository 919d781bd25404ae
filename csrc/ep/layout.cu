// Token-layout and count-exchange ("notify") kernels of normal-mode dispatch.
//
// Replaces what the reference obtains from DeepEP's `Buffer.get_dispatch_layout` and the
// count exchange hidden inside `Buffer.dispatch` (`DeepEP_v1/deepep_v1_dispatch.py:199-230`):
// per-rank / per-expert token counts, `is_token_in_rank`, stable positions of every item in
// its (source rank -> bucket) stream, and an all-gather of the count vectors over NVLink with
// plain peer stores + release flags. The prefix sums that turn the gathered counts into the
// exact destination row of every token are computed by every CTA of the dispatch kernel itself
// (csrc/ep/dispatch.cu), so the count exchange costs one small launch, not two.
#include <cooperative_groups.h>

#include "ep.cuh"
#include "api.h"

namespace cg = cooperative_groups;

namespace b200ep {

// ---------------------------------------------------------------------------------------
// layout: counts + is_token_in_rank. One thread per token, shared-memory histograms per CTA,
// per-CTA partial histograms in a scratch matrix, summed by the last CTA: the outputs need no
// zero-fill before the launch and the sums do not depend on the order of atomics.
// ---------------------------------------------------------------------------------------
constexpr int kLayoutThreads = 256;
// One cluster of 8 CTAs covers the token counts an EP step sees (a grid-stride loop takes the
// rest); beyond kLayoutClusterMaxTokens the multi-CTA kernel with a last-CTA sum runs instead.
constexpr int kSmallCluster = 8;
constexpr int kSmallClusterThreads = 512;
constexpr int kLayoutClusterMaxTokens = 1 << 16;

// Histogram contribution and is_token_in_rank row of one token; he/hr are shared-memory
// histograms over experts / ranks.
__device__ __forceinline__ void layout_token(const long long* __restrict__ topk_idx, int t, int K,
                                             int E, int R, int El, int* he, int* hr,
                                             bool* __restrict__ is_token_in_rank, int* status) {
  unsigned mask = 0;
  for (int k0 = 0; k0 < K; k0 += 8) {
    long long e[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) e[u] = (k0 + u < K) ? topk_idx[(size_t)t * K + k0 + u] : -1;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      if (e[u] >= 0 && e[u] < E) {
        atomicAdd(&he[(int)e[u]], 1);
        mask |= 1u << ((int)e[u] / El);
      } else if (e[u] != -1) {
        set_status(status, kBadExpertIndex);
      }
    }
  }
  for (int d = 0; d < R; ++d) {
    const bool in = (mask >> d) & 1u;
    is_token_in_rank[(size_t)t * R + d] = in;
    if (in) atomicAdd(&hr[d], 1);
  }
}

__global__ void __launch_bounds__(kLayoutThreads)
layout_kernel(const long long* __restrict__ topk_idx, int T, int K, int E, int R,
              int* __restrict__ num_tokens_per_rank, int* __restrict__ num_tokens_per_expert,
              bool* __restrict__ is_token_in_rank, int* partial, unsigned int* block_counter,
              int* status) {
  extern __shared__ int sh[];
  int* he = sh;
  int* hr = sh + E;
  for (int i = threadIdx.x; i < E + R; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < T) layout_token(topk_idx, t, K, E, R, E / R, he, hr, is_token_in_rank, status);
  __syncthreads();
  const int V = E + R;
  if (gridDim.x == 1) {
    for (int i = threadIdx.x; i < E; i += blockDim.x) num_tokens_per_expert[i] = he[i];
    for (int i = threadIdx.x; i < R; i += blockDim.x) num_tokens_per_rank[i] = hr[i];
    return;
  }
  for (int i = threadIdx.x; i < V; i += blockDim.x) partial[(size_t)blockIdx.x * V + i] = sh[i];
  if (!last_block_arrive(block_counter, gridDim.x)) return;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    int s = 0;
    for (unsigned int b = 0; b < gridDim.x; ++b) s += __ldcg(&partial[(size_t)b * V + i]);
    if (i < E) num_tokens_per_expert[i] = s;
    else num_tokens_per_rank[i - E] = s;
  }
}

// The same work as ONE thread-block cluster: every CTA builds its histogram in its own shared
// memory, a cluster barrier replaces the partial matrix + device fence + arrival counter, and
// CTA 0 sums the eight histograms through distributed shared memory. The second barrier keeps
// the other CTAs (and their shared memory) alive until CTA 0 has read them.
__global__ void __cluster_dims__(kSmallCluster, 1, 1) __launch_bounds__(kSmallClusterThreads, 1)
layout_cluster_kernel(const long long* __restrict__ topk_idx, int T, int K, int E, int R,
                      int* __restrict__ num_tokens_per_rank, int* __restrict__ num_tokens_per_expert,
                      bool* __restrict__ is_token_in_rank, int* status) {
  extern __shared__ int sh[];
  cg::cluster_group cluster = cg::this_cluster();
  int* he = sh;
  int* hr = sh + E;
  for (int i = threadIdx.x; i < E + R; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const int El = E / R;
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < T; t += gridDim.x * blockDim.x)
    layout_token(topk_idx, t, K, E, R, El, he, hr, is_token_in_rank, status);
  cluster.sync();
  if (cluster.block_rank() == 0) {
    for (int i = threadIdx.x; i < E + R; i += blockDim.x) {
      int s = 0;
#pragma unroll
      for (int r = 0; r < kSmallCluster; ++r) s += cluster.map_shared_rank(sh, r)[i];
      if (i < E) num_tokens_per_expert[i] = s;
      else num_tokens_per_rank[i - E] = s;
    }
  }
  cluster.sync();
}

int layout_scratch_ints(int T, int E, int R) {
  const int blocks = T > 0 ? (T + kLayoutThreads - 1) / kLayoutThreads : 1;
  return blocks * (E + R);
}

void launch_layout(const long long* topk_idx, int T, int K, int E, int R, int* per_rank,
                   int* per_expert, bool* in_rank, int* partial, unsigned int* block_counter,
                   int* status, cudaStream_t st) {
  const size_t smem = (E + R) * sizeof(int);
  if (T > kLayoutThreads && T <= kLayoutClusterMaxTokens && smem <= 48 * 1024) {
    layout_cluster_kernel<<<kSmallCluster, kSmallClusterThreads, smem, st>>>(
        topk_idx, T, K, E, R, per_rank, per_expert, in_rank, status);
    return;
  }
  const int blocks = T > 0 ? (T + kLayoutThreads - 1) / kLayoutThreads : 1;
  layout_kernel<<<blocks, kLayoutThreads, smem, st>>>(
      topk_idx, T, K, E, R, per_rank, per_expert, in_rank, partial, block_counter, status);
}

// ---------------------------------------------------------------------------------------
// notify_send: one WARP per chunk of 32 tokens (lane = token) computes the stable rank of each
// item inside its chunk and the chunk histogram:
//   rank mode   : for every destination rank one ballot over the chunk's tokens;
//   expert mode : a 32-bit mask per expert in shared memory (bit = token of the chunk that
//                 chose the expert); an item's rank is the number of lower bits.
// The last CTA to finish scans the histograms over chunks (turning them into chunk bases),
// builds this rank's count vector [R rank counts | E expert counts], stores it into every
// peer's count matrix and releases the notify flag.
// ---------------------------------------------------------------------------------------
constexpr int kNotifyWarps = 8;

// One chunk of 32 tokens (lane = token) by one warp. `bits` is the warp's [B] bitmask scratch in
// shared memory (expert mode only).
template <int MODE>
__device__ __forceinline__ void notify_chunk(const EpGeom& g, int c, int lane, unsigned int* bits,
                                             const bool* __restrict__ is_in_rank,
                                             const long long* __restrict__ topk_idx,
                                             int* __restrict__ item_rank, int* chunk_hist,
                                             int* status) {
  const int J = g.J, B = g.B, R = g.R, E = g.E, K = g.K;
  const unsigned lt = (1u << lane) - 1u;
  const int t = c * kChunkTokens + lane;
  const bool valid = t < g.T;
  if (MODE == 0) {
    // all R flags of my token first (independent loads, one latency), then one ballot per rank
    unsigned mine = 0;
    if (valid)
      for (int j = 0; j < R; ++j) mine |= (is_in_rank[(size_t)t * R + j] ? 1u : 0u) << j;
    for (int j = 0; j < R; ++j) {
      const bool in = (mine >> j) & 1u;
      const unsigned m = __ballot_sync(0xffffffffu, in);
      if (valid) item_rank[(size_t)t * J + j] = in ? __popc(m & lt) : -1;
      if (lane == 0) chunk_hist[(size_t)c * B + j] = __popc(m);
    }
  } else {
    for (int b = lane; b < B; b += 32) bits[b] = 0u;
    __syncwarp();
    bool dup = false;
    for (int k = 0; k < K; ++k) {
      const long long e = valid ? topk_idx[(size_t)t * K + k] : -1;
      if (e >= 0 && e < E) {
        const unsigned old = atomicOr(&bits[(int)e], 1u << lane);
        if (old & (1u << lane)) dup = true;     // the same expert twice in one token
      } else if (e != -1) {
        set_status(status, kBadExpertIndex);
      }
    }
    if (dup) set_status(status, kBadExpertIndex);
    __syncwarp();
    for (int k = 0; k < K && valid; ++k) {
      const long long e = topk_idx[(size_t)t * K + k];
      int r = -1;
      if (e >= 0 && e < E) {
        r = __popc(bits[(int)e] & lt);
        if (dup)                                 // keep the first occurrence only
          for (int q = 0; q < k; ++q)
            if (topk_idx[(size_t)t * K + q] == e) r = -1;
      }
      item_rank[(size_t)t * J + k] = r;
    }
    for (int b = lane; b < B; b += 32) chunk_hist[(size_t)c * B + b] = __popc(bits[b]);
    __syncwarp();
  }
}

// Run by ONE CTA after every chunk histogram is visible to it: exclusive scan over chunks per
// bucket (histograms become chunk bases), this rank's count vector, its copy into every peer's
// count matrix, and the notify flag. `hist` is [B + R + E] ints of shared memory.
// The flag store is a system-scope release issued after a CTA barrier that follows the count
// stores, which orders them before the flag for every observer (release cumulativity).
template <int MODE>
__device__ __forceinline__ void notify_publish(const EpGeom& g, const EpRegions& rg,
                                               const PeerPtrs& peers,
                                               const int* __restrict__ num_tokens_per_expert,
                                               int* chunk_hist, int* hist, int C) {
  const int B = g.B, R = g.R, E = g.E;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  int* vec = hist + B;                                   // [R+E]
  if (B <= nwarps * 2) {
    // few buckets: one warp per bucket, lanes over chunks, all loads of a pass issued together
    for (int b = warp; b < B; b += nwarps) {
      int carry = 0;
      for (int c0 = 0; c0 < C; c0 += 128) {
        int v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int cc = c0 + u * 32 + lane;
          v[u] = cc < C ? __ldcg(&chunk_hist[(size_t)cc * B + b]) : 0;
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int cc = c0 + u * 32 + lane;
          int incl = v[u];
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
          }
          if (cc < C) chunk_hist[(size_t)cc * B + b] = carry + incl - v[u];
          carry += __shfl_sync(0xffffffffu, incl, 31);
        }
      }
      if (lane == 0) hist[b] = carry;
    }
  } else {
    // many buckets: one thread per bucket (coalesced across buckets), chunks in batches of
    // independent loads
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
      int carry = 0;
      for (int c0 = 0; c0 < C; c0 += 16) {
        int v[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) v[u] = (c0 + u < C) ? __ldcg(&chunk_hist[(size_t)(c0 + u) * B + b]) : 0;
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          if (c0 + u < C) chunk_hist[(size_t)(c0 + u) * B + b] = carry;
          carry += v[u];
        }
      }
      hist[b] = carry;
    }
  }
  __syncthreads();
  const int V = R + E;
  if (MODE == 0) {
    for (int i = threadIdx.x; i < R; i += blockDim.x) vec[i] = hist[i];
    for (int i = threadIdx.x; i < E; i += blockDim.x)
      vec[R + i] = num_tokens_per_expert ? num_tokens_per_expert[i] : 0;
  } else {
    for (int i = threadIdx.x; i < E; i += blockDim.x) vec[R + i] = hist[i];
    for (int d = threadIdx.x; d < R; d += blockDim.x) {
      int s = 0;
      for (int q = 0; q < g.El; ++q) s += hist[d * g.El + q];
      vec[d] = s;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < R * V; i += blockDim.x) {
    const int p = i / V, v = i % V;
    int* dst = reinterpret_cast<int*>(peers.base[p] + rg.counts) + (size_t)g.rank * V + v;
    st_relaxed_sys(dst, vec[v]);
  }
  __syncthreads();
  if (threadIdx.x < R) {
    int* flag = reinterpret_cast<int*>(peers.base[threadIdx.x] + rg.flags) +
                kChNotify * kMaxRanks + g.rank;
    st_release_sys(flag, g.epoch);
  }
}

template <int MODE>
__global__ void __launch_bounds__(kNotifyWarps * 32)
notify_send_kernel(EpGeom g, EpRegions rg, PeerPtrs peers, const bool* __restrict__ is_in_rank,
                   const long long* __restrict__ topk_idx,
                   const int* __restrict__ num_tokens_per_expert, int* __restrict__ item_rank,
                   int* chunk_hist, unsigned int* block_counter, int* status) {
  extern __shared__ int sh[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int C = g.T > 0 ? (g.T + kChunkTokens - 1) / kChunkTokens : 1;
  const int c = blockIdx.x * kNotifyWarps + warp;
  if (c < C)
    notify_chunk<MODE>(g, c, lane, reinterpret_cast<unsigned int*>(sh) + (size_t)warp * g.B,
                       is_in_rank, topk_idx, item_rank, chunk_hist, status);
  if (!last_block_arrive(block_counter, gridDim.x)) return;
  notify_publish<MODE>(g, rg, peers, num_tokens_per_expert, chunk_hist,
                       sh + (MODE == 1 ? kNotifyWarps * g.B : 0), C);
}

// One thread-block cluster instead of a grid with an arrival counter: the warps of the eight
// CTAs stride over the chunks, a cluster barrier (release/acquire at cluster scope, which
// covers the global-memory histograms the other CTAs wrote) replaces the device fence + atomic,
// and CTA 0 publishes.
template <int MODE>
__global__ void __cluster_dims__(kSmallCluster, 1, 1) __launch_bounds__(kSmallClusterThreads)
notify_send_cluster_kernel(EpGeom g, EpRegions rg, PeerPtrs peers,
                           const bool* __restrict__ is_in_rank,
                           const long long* __restrict__ topk_idx,
                           const int* __restrict__ num_tokens_per_expert,
                           int* __restrict__ item_rank, int* chunk_hist, int* status) {
  extern __shared__ int sh[];
  constexpr int kWarps = kSmallClusterThreads / 32;
  cg::cluster_group cluster = cg::this_cluster();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int C = g.T > 0 ? (g.T + kChunkTokens - 1) / kChunkTokens : 1;
  for (int c = blockIdx.x * kWarps + warp; c < C; c += gridDim.x * kWarps)
    notify_chunk<MODE>(g, c, lane, reinterpret_cast<unsigned int*>(sh) + (size_t)warp * g.B,
                       is_in_rank, topk_idx, item_rank, chunk_hist, status);
  cluster.sync();
  if (cluster.block_rank() != 0) return;
  notify_publish<MODE>(g, rg, peers, num_tokens_per_expert, chunk_hist,
                       sh + (MODE == 1 ? kWarps * g.B : 0), C);
}

void launch_notify_send(const EpGeom& g, const EpRegions& rg, const PeerPtrs& peers,
                        const bool* is_in_rank, const long long* topk_idx,
                        const int* num_tokens_per_expert, int* item_rank, int* chunk_hist,
                        unsigned int* block_counter, int* status, cudaStream_t st) {
  const int C = g.T > 0 ? (g.T + kChunkTokens - 1) / kChunkTokens : 1;
  constexpr int kClusterWarps = kSmallClusterThreads / 32;
  const size_t csmem = sizeof(int) * ((g.mode == 1 ? kClusterWarps * g.B : 0) + g.B + g.R + g.E);
  if (C > kNotifyWarps && C <= kLayoutClusterMaxTokens / kChunkTokens && csmem <= 200 * 1024) {
    if (g.mode == 0) {
      notify_send_cluster_kernel<0><<<kSmallCluster, kSmallClusterThreads, csmem, st>>>(
          g, rg, peers, is_in_rank, topk_idx, num_tokens_per_expert, item_rank, chunk_hist, status);
    } else {
      if (csmem > 48 * 1024)
        cudaFuncSetAttribute(notify_send_cluster_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)csmem);
      notify_send_cluster_kernel<1><<<kSmallCluster, kSmallClusterThreads, csmem, st>>>(
          g, rg, peers, is_in_rank, topk_idx, num_tokens_per_expert, item_rank, chunk_hist, status);
    }
    return;
  }
  const int blocks = (C + kNotifyWarps - 1) / kNotifyWarps;
  const size_t smem = sizeof(int) * ((g.mode == 1 ? kNotifyWarps * g.B : 0) + g.B + g.R + g.E);
  if (g.mode == 0) {
    notify_send_kernel<0><<<blocks, kNotifyWarps * 32, smem, st>>>(
        g, rg, peers, is_in_rank, topk_idx, num_tokens_per_expert, item_rank, chunk_hist,
        block_counter, status);
  } else {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(notify_send_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    notify_send_kernel<1><<<blocks, kNotifyWarps * 32, smem, st>>>(
        g, rg, peers, is_in_rank, topk_idx, num_tokens_per_expert, item_rank, chunk_hist,
        block_counter, status);
  }
}

// ---------------------------------------------------------------------------------------
// Generic bounded wait on one flag channel (all ranks), and the self-test wait.
// ---------------------------------------------------------------------------------------
__global__ void wait_flags_kernel(const int* flags, int R, int epoch, unsigned long long timeout_ns,
                                  int* status, int code) {
  if (threadIdx.x < R) wait_flag_ge(flags + threadIdx.x, epoch, timeout_ns, status, code);
}

void launch_wait_flags(char* self_base, long long flags_off, int channel, int R, int epoch,
                       unsigned long long timeout_ns, int* status, int code, cudaStream_t st) {
  const int* flags = reinterpret_cast<const int*>(self_base + flags_off) + channel * kMaxRanks;
  wait_flags_kernel<<<1, 32, 0, st>>>(flags, R, epoch, timeout_ns, status, code);
}

// Barrier across ranks: publish epoch on every peer's barrier channel, wait for all.
__global__ void barrier_kernel(PeerPtrs peers, long long flags_off, int rank, int R, int epoch,
                               unsigned long long timeout_ns, int* status, int wait) {
  if (threadIdx.x < R) {
    fence_acq_rel_sys();
    int* remote = reinterpret_cast<int*>(peers.base[threadIdx.x] + flags_off) +
                  kChBarrier * kMaxRanks + rank;
    st_release_sys(remote, epoch);
    if (wait) {
      const int* mine = reinterpret_cast<const int*>(peers.base[rank] + flags_off) +
                        kChBarrier * kMaxRanks + threadIdx.x;
      wait_flag_ge(mine, epoch, timeout_ns, status, kTimeoutBarrier);
    }
  }
}

void launch_barrier(const PeerPtrs& peers, long long flags_off, int rank, int R, int epoch,
                    unsigned long long timeout_ns, int* status, int wait, cudaStream_t st) {
  barrier_kernel<<<1, 32, 0, st>>>(peers, flags_off, rank, R, epoch, timeout_ns, status, wait);
}

}  // namespace b200ep
