// Token-layout and count-exchange ("notify") kernels of normal-mode dispatch.
//
// Replaces what the reference obtains from DeepEP's `Buffer.get_dispatch_layout` and the
// count exchange hidden inside `Buffer.dispatch` (`DeepEP_v1/deepep_v1_dispatch.py:199-230`):
// per-rank / per-expert token counts, `is_token_in_rank`, stable positions of every item in
// its (source rank -> bucket) stream, an all-gather of the count vectors over NVLink with
// plain peer stores + release flags, and the prefix sums that give every sender the exact
// destination row of every token (so payload is stored once, in its final place).
#include "ep.cuh"
#include "api.h"

namespace b200ep {

// ---------------------------------------------------------------------------------------
// layout: counts + is_token_in_rank. One thread per token, shared-memory histograms.
// ---------------------------------------------------------------------------------------
__global__ void layout_kernel(const long long* __restrict__ topk_idx, int T, int K, int E, int R,
                              int* __restrict__ num_tokens_per_rank,
                              int* __restrict__ num_tokens_per_expert,
                              bool* __restrict__ is_token_in_rank, int* status) {
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
  for (int i = threadIdx.x; i < E; i += blockDim.x)
    if (he[i]) atomicAdd(&num_tokens_per_expert[i], he[i]);
  for (int i = threadIdx.x; i < R; i += blockDim.x)
    if (hr[i]) atomicAdd(&num_tokens_per_rank[i], hr[i]);
}

void launch_layout(const long long* topk_idx, int T, int K, int E, int R, int* per_rank,
                   int* per_expert, bool* in_rank, int* status, cudaStream_t st) {
  if (per_expert == per_rank + R) {
    cudaMemsetAsync(per_rank, 0, sizeof(int) * (R + E), st);   // one buffer: [R rank counts | E expert counts]
  } else {
    cudaMemsetAsync(per_rank, 0, sizeof(int) * R, st);
    cudaMemsetAsync(per_expert, 0, sizeof(int) * E, st);
  }
  if (T == 0) return;
  const int threads = 256;
  layout_kernel<<<(T + threads - 1) / threads, threads, (E + R) * sizeof(int), st>>>(
      topk_idx, T, K, E, R, per_rank, per_expert, in_rank, status);
}

// ---------------------------------------------------------------------------------------
// notify_send: one CTA per chunk of 32 tokens computes the stable intra-chunk rank of each
// item and the chunk histogram; the last CTA to finish scans the histograms over chunks
// (turning them into chunk bases), builds this rank's count vector [R rank counts | E expert
// counts] and stores it into every peer's count matrix, then releases the notify flag.
// ---------------------------------------------------------------------------------------
template <int MODE>
__global__ void notify_send_kernel(EpGeom g, EpRegions rg, PeerPtrs peers,
                                   const bool* __restrict__ is_in_rank,
                                   const long long* __restrict__ topk_idx,
                                   const int* __restrict__ num_tokens_per_expert,
                                   int* __restrict__ item_rank, int* chunk_hist,
                                   unsigned int* block_counter, int* status) {
  extern __shared__ int sh[];
  const int J = g.J, B = g.B, R = g.R, E = g.E;
  int* items = sh;                       // [32*J]
  int* hist = sh + kChunkTokens * J;     // [B]
  int* vec = hist + B;                   // [R+E]
  const int n_items = kChunkTokens * J;
  const int c = blockIdx.x;
  const int t0 = c * kChunkTokens;

  for (int i = threadIdx.x; i < B; i += blockDim.x) hist[i] = 0;
  for (int i = threadIdx.x; i < n_items; i += blockDim.x) {
    const int t = t0 + i / J, j = i % J;
    int b = -1;
    if (t < g.T) {
      if (MODE == 0) {
        b = is_in_rank[(size_t)t * R + j] ? j : -1;
      } else {
        const long long e = topk_idx[(size_t)t * g.K + j];
        b = (e >= 0 && e < E) ? (int)e : -1;
      }
    }
    items[i] = b;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_items; i += blockDim.x) {
    const int b = items[i];
    int r = -1;
    if (b >= 0) {
      r = 0;
      for (int q = 0; q < i; ++q) r += (items[q] == b);
      atomicAdd(&hist[b], 1);
    }
    const int t = t0 + i / J;
    if (t < g.T) item_rank[(size_t)t * J + i % J] = r;
  }
  __syncthreads();
  for (int b = threadIdx.x; b < B; b += blockDim.x) chunk_hist[(size_t)c * B + b] = hist[b];

  if (!last_block_arrive(block_counter, gridDim.x)) return;

  // ---- last block: exclusive scan over chunks, per bucket (one warp per bucket, 32 chunks per
  // step, coalesced loads issued together; a serial loop here costs one L2 round trip per chunk) ----
  const int C = gridDim.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int b = warp; b < B; b += nwarps) {
    int carry = 0;
    for (int c0 = 0; c0 < C; c0 += 32) {
      const int cc = c0 + lane;
      const int v = cc < C ? __ldcg(&chunk_hist[(size_t)cc * B + b]) : 0;
      int incl = v;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
      }
      if (cc < C) chunk_hist[(size_t)cc * B + b] = carry + incl - v;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) hist[b] = carry;  // total per bucket
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
  int threads = kChunkTokens * g.J;
  if (threads < 256) threads = 256;
  if (threads > 1024) threads = 1024;
  const size_t smem = sizeof(int) * (kChunkTokens * g.J + g.B + g.R + g.E);
  if (g.mode == 0)
    notify_send_kernel<0><<<C, threads, smem, st>>>(g, rg, peers, is_in_rank, topk_idx,
                                                    num_tokens_per_expert, item_rank, chunk_hist,
                                                    block_counter, status);
  else
    notify_send_kernel<1><<<C, threads, smem, st>>>(g, rg, peers, is_in_rank, topk_idx,
                                                    num_tokens_per_expert, item_rank, chunk_hist,
                                                    block_counter, status);
}

// ---------------------------------------------------------------------------------------
// notify_wait: one CTA. Waits (bounded) for every peer's count vector, then derives
//   send_base[b]  row in the destination where my stream for bucket b starts,
//   comb_base[b]  slot in MY combine region where results for bucket b start,
//   recv offsets / counts on my side, and publishes N_recv + per-expert counts to pinned
//   host memory so the host can size the output tensors without a device synchronise.
// ---------------------------------------------------------------------------------------
__global__ void notify_wait_kernel(EpGeom g, EpRegions rg, char* self_base, EpMeta m,
                                   volatile int* host_word, int* status) {
  extern __shared__ int col[];  // [E] column totals
  __shared__ int ok;
  const int R = g.R, E = g.E, El = g.El, V = g.R + g.E, me = g.rank;
  const int* flags = reinterpret_cast<const int*>(self_base + rg.flags) + kChNotify * kMaxRanks;
  const int* M = reinterpret_cast<const int*>(self_base + rg.counts);
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < R) {
    if (!wait_flag_ge(flags + threadIdx.x, g.epoch, g.timeout_ns, status, kTimeoutNotify)) ok = 0;
  }
  __syncthreads();
  if (!ok) {
    if (threadIdx.x == 0) {
      *m.n_recv = 0;
      *m.send_total = -1;      // tells dispatch_send that the offsets are not valid: send nothing
      host_word[1] = -1;
      __threadfence_system();
      host_word[0] = g.epoch;
    }
    return;
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int s = 0;
    for (int r = 0; r < R; ++r) s += __ldcg(&M[r * V + R + e]);
    col[e] = s;
  }
  __syncthreads();
  if (g.mode == 0) {
    for (int d = threadIdx.x; d < R; d += blockDim.x) {
      int sb = 0, cb = 0;
      for (int s = 0; s < me; ++s) sb += __ldcg(&M[s * V + d]);
      for (int q = 0; q < d; ++q) cb += __ldcg(&M[me * V + q]);
      m.send_base[d] = sb;
      m.comb_base[d] = cb;
    }
  } else {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      const int d = e / El, gl = e % El;
      int sb = 0, cb = 0;
      for (int q = 0; q < gl; ++q) sb += col[d * El + q];
      for (int s = 0; s < me; ++s) sb += __ldcg(&M[s * V + R + e]);
      for (int q = 0; q < e; ++q) cb += __ldcg(&M[me * V + R + q]);
      m.send_base[e] = sb;
      m.comb_base[e] = cb;
    }
  }
  if (threadIdx.x == 0) {
    int n_recv = 0, acc = 0, stot = 0;
    for (int s = 0; s < R; ++s) {
      m.recv_src_off[s] = n_recv;
      n_recv += __ldcg(&M[s * V + me]);
    }
    m.recv_src_off[R] = n_recv;
    for (int q = 0; q < El; ++q) {
      const int cnt = col[me * El + q];
      m.recv_expert_cnt[q] = cnt;
      m.recv_expert_off[q] = acc;
      acc += cnt;
      host_word[2 + q] = cnt;
    }
    m.recv_expert_off[El] = acc;
    if (g.mode == 1) {
      n_recv = acc;
      for (int q = 0; q < E; ++q) stot += __ldcg(&M[me * V + R + q]);
    } else {
      for (int q = 0; q < R; ++q) stot += __ldcg(&M[me * V + q]);
    }
    *m.n_recv = n_recv;
    *m.send_total = stot;
    if (n_recv > g.cap) set_status(status, kOverflowRecv);
    if (stot > g.slot_cap) set_status(status, kOverflowSlots);
    host_word[1] = n_recv;
    __threadfence_system();
    host_word[0] = g.epoch;
  }
}

void launch_notify_wait(const EpGeom& g, const EpRegions& rg, char* self_base, const EpMeta& m,
                        int* host_word, int* status, cudaStream_t st) {
  notify_wait_kernel<<<1, 256, sizeof(int) * g.E, st>>>(g, rg, self_base, m, host_word, status);
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
