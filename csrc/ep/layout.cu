// Token-layout and count-exchange ("notify") kernels of normal-mode dispatch.
//
// Replaces what the reference obtains from DeepEP's `Buffer.get_dispatch_layout` and the
// count exchange hidden inside `Buffer.dispatch` (`DeepEP_v1/deepep_v1_dispatch.py:199-230`):
// per-rank / per-expert token counts, `is_token_in_rank`, stable positions of every item in
// its (source rank -> bucket) stream, and an all-gather of the count vectors over NVLink with
// plain peer stores + release flags. The prefix sums that turn the gathered counts into the
// exact destination row of every token are computed by every CTA of the dispatch kernel itself
// (csrc/ep/dispatch.cu), so the count exchange costs one small launch, not two.
#include "ep.cuh"
#include "api.h"

namespace b200ep {

// ---------------------------------------------------------------------------------------
// layout: counts + is_token_in_rank. One thread per token, shared-memory histograms per CTA,
// per-CTA partial histograms in a scratch matrix, summed by the last CTA: the outputs need no
// zero-fill before the launch and the sums do not depend on the order of atomics.
// ---------------------------------------------------------------------------------------
constexpr int kLayoutThreads = 256;

__global__ void __launch_bounds__(kLayoutThreads)
layout_kernel(const long long* __restrict__ topk_idx, int T, int K, int E, int R,
              int* __restrict__ num_tokens_per_rank, int* __restrict__ num_tokens_per_expert,
              bool* __restrict__ is_token_in_rank, int* partial, unsigned int* block_counter,
              int* status) {
  extern __shared__ int sh[];
  int* he = sh;
  int* hr = sh + E;
  const int El = E / R;
  for (int i = threadIdx.x; i < E + R; i += blockDim.x) sh[i] = 0;
  __syncthreads();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t < T) {
    unsigned mask = 0;
    for (int k = 0; k < K; ++k) {
      const long long e = topk_idx[(size_t)t * K + k];
      if (e >= 0 && e < E) {
        atomicAdd(&he[(int)e], 1);
        mask |= 1u << ((int)e / El);
      } else if (e != -1) {
        set_status(status, kBadExpertIndex);
      }
    }
    for (int d = 0; d < R; ++d) {
      const bool in = (mask >> d) & 1u;
      is_token_in_rank[(size_t)t * R + d] = in;
      if (in) atomicAdd(&hr[d], 1);
    }
  }
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

int layout_scratch_ints(int T, int E, int R) {
  const int blocks = T > 0 ? (T + kLayoutThreads - 1) / kLayoutThreads : 1;
  return blocks * (E + R);
}

void launch_layout(const long long* topk_idx, int T, int K, int E, int R, int* per_rank,
                   int* per_expert, bool* in_rank, int* partial, unsigned int* block_counter,
                   int* status, cudaStream_t st) {
  const int blocks = T > 0 ? (T + kLayoutThreads - 1) / kLayoutThreads : 1;
  layout_kernel<<<blocks, kLayoutThreads, (E + R) * sizeof(int), st>>>(
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

template <int MODE>
__global__ void __launch_bounds__(kNotifyWarps * 32)
notify_send_kernel(EpGeom g, EpRegions rg, PeerPtrs peers, const bool* __restrict__ is_in_rank,
                   const long long* __restrict__ topk_idx,
                   const int* __restrict__ num_tokens_per_expert, int* __restrict__ item_rank,
                   int* chunk_hist, unsigned int* block_counter, int* status) {
  extern __shared__ int sh[];
  const int J = g.J, B = g.B, R = g.R, E = g.E, K = g.K;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const unsigned lt = (1u << lane) - 1u;
  const int C = g.T > 0 ? (g.T + kChunkTokens - 1) / kChunkTokens : 1;
  const int c = blockIdx.x * kNotifyWarps + warp;
  if (c < C) {
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
      unsigned int* bits = reinterpret_cast<unsigned int*>(sh) + (size_t)warp * B;
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
    }
  }

  if (!last_block_arrive(block_counter, gridDim.x)) return;

  // ---- last block: exclusive scan over chunks, per bucket -------------------------------
  int* hist = sh + (MODE == 1 ? kNotifyWarps * B : 0);   // [B] totals
  int* vec = hist + B;                                   // [R+E]
  if (B <= kNotifyWarps * 2) {
    // few buckets: one warp per bucket, lanes over chunks, all loads of a pass issued together
    for (int b = warp; b < B; b += kNotifyWarps) {
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
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < R) {
    int* flag = reinterpret_cast<int*>(peers.base[threadIdx.x] + rg.flags) +
                kChNotify * kMaxRanks + g.rank;
    st_release_sys(flag, g.epoch);
  }
}

void launch_notify_send(const EpGeom& g, const EpRegions& rg, const PeerPtrs& peers,
                        const bool* is_in_rank, const long long* topk_idx,
                        const int* num_tokens_per_expert, int* item_rank, int* chunk_hist,
                        unsigned int* block_counter, int* status, cudaStream_t st) {
  const int C = g.T > 0 ? (g.T + kChunkTokens - 1) / kChunkTokens : 1;
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
