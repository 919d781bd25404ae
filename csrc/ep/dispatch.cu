// Normal-mode dispatch: ONE kernel reads each local token once, optionally casts it to
// block-scaled fp8 (e4m3, one f32 scale per 128 channels), and stores it straight into its
// final row of every destination rank's receive region over NVLink with 16-byte LSU peer
// stores. The permute is part of the address computation, so no separate permute kernel and
// no staging ring exist. Replaces `Buffer.dispatch` as consumed by
// `DeepEP_v1/deepep_v1_dispatch.py:212-230` and, in expert mode, also the multihot/permute
// glue of `DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:276-388`.
//
// Structure of one launch:
//   prologue (every CTA)  bounded wait for the peers' count vectors, then the prefix sums that
//                         give, per bucket, the first row at the destination (`send_base`) and
//                         the first slot of this rank's combine region (`comb_base`), kept in
//                         shared memory. CTA 0 also writes the receive-side tables of the
//                         handle and the receive count for the host.
//   body                  one warp per token, 16-byte stores to every destination.
//   epilogue (last CTA)   release this rank's dispatch flag on every peer; when the kernel is
//                         not one of several virtual ranks on one GPU, also wait (bounded) for
//                         the peers' flags, so the receive region is complete when it ends.
#include <cuda_bf16.h>
#include "cast.cuh"
#include "ep.cuh"
#include "api.h"

namespace b200ep {

constexpr int kSendWarps = 16;  // warps per CTA in the send kernels
constexpr int kUnroll = 4;

// Exclusive prefix sum of a[0..n) in place by ONE warp (n is a few hundred at most).
__device__ __forceinline__ void warp_exclusive_scan(int* a, int n, int lane) {
  int carry = 0;
  for (int i0 = 0; i0 < n; i0 += 32) {
    const int i = i0 + lane;
    const int v = i < n ? a[i] : 0;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int x = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += x;
    }
    if (i < n) a[i] = carry + incl - v;
    carry += __shfl_sync(0xffffffffu, incl, 31);
  }
}

// Waits for the count vectors of notify epoch g.epoch_wait and fills s_send_base[B],
// s_comb_base[B] (shared memory). `scratch` holds E ints. Returns false after a time-out.
__device__ bool dispatch_prologue(const EpGeom& g, const EpRegions& rg, char* self_base,
                                  int* s_send_base, int* s_comb_base, int* scratch, int* status) {
  __shared__ int s_ok;
  const int R = g.R, E = g.E, El = g.El, V = g.R + g.E, me = g.rank;
  const int* flags = reinterpret_cast<const int*>(self_base + rg.flags) + kChNotify * kMaxRanks;
  const int* M = reinterpret_cast<const int*>(self_base + rg.counts);
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < R) {
    if (!wait_flag_ge(flags + threadIdx.x, g.epoch_wait, g.timeout_ns, status, kTimeoutNotify)) s_ok = 0;
  }
  __syncthreads();
  if (!s_ok) return false;
  if (g.mode == 0) {
    if ((int)threadIdx.x < R) {
      const int d = threadIdx.x;
      int sb = 0, cb = 0;
      for (int s = 0; s < me; ++s) sb += __ldcg(&M[s * V + d]);
      for (int q = 0; q < d; ++q) cb += __ldcg(&M[me * V + q]);
      s_send_base[d] = sb;
      s_comb_base[d] = cb;
    }
  } else {
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      int col = 0, part = 0;
      for (int r = 0; r < R; ++r) {
        const int v = __ldcg(&M[r * V + R + e]);
        col += v;
        if (r < me) part += v;
      }
      scratch[e] = col;                               // rows that expert e receives in total
      s_send_base[e] = part;                          // ... of which from lower source ranks
      s_comb_base[e] = __ldcg(&M[me * V + R + e]);    // my own count for e
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      warp_exclusive_scan(scratch, E, threadIdx.x);
      warp_exclusive_scan(s_comb_base, E, threadIdx.x);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x)
      s_send_base[e] += scratch[e] - scratch[(e / El) * El];   // prefix inside the destination rank
  }
  __syncthreads();
  return true;
}

// CTA 0 only: receive-side tables of the handle, host words, overflow checks.
__device__ void dispatch_publish_meta(const EpGeom& g, const EpRegions& rg, const PeerPtrs& peers,
                                      char* self_base, const EpMeta& m, const int* s_send_base,
                                      const int* s_comb_base, volatile int* host_word, int* status,
                                      bool ok) {
  __shared__ int s_cnt[kMaxRanks + 1];
  const int R = g.R, E = g.E, El = g.El, V = g.R + g.E, me = g.rank, B = g.B;
  if (!ok) {
    if (threadIdx.x == 0) {
      *m.n_recv = 0;
      *m.send_total = -1;
      if (host_word) {
        host_word[1] = -1;
        __threadfence_system();
        host_word[0] = g.epoch_wait;
      }
    }
    return;
  }
  const int* M = reinterpret_cast<const int*>(self_base + rg.counts);
  for (int b = threadIdx.x; b < B; b += blockDim.x) {
    m.send_base[b] = s_send_base[b];
    m.comb_base[b] = s_comb_base[b];
  }
  for (int q = threadIdx.x; q < El; q += blockDim.x) {
    int cnt = 0;
    for (int r = 0; r < R; ++r) cnt += __ldcg(&M[r * V + R + me * El + q]);
    m.recv_expert_cnt[q] = cnt;
    if (host_word) host_word[2 + q] = cnt;
  }
  if ((int)threadIdx.x < R) s_cnt[threadIdx.x] = __ldcg(&M[threadIdx.x * V + me]);
  __syncthreads();
  if (threadIdx.x == 0) {
    int n_recv = 0, acc = 0, stot = 0;
    for (int s = 0; s < R; ++s) {
      m.recv_src_off[s] = n_recv;
      n_recv += s_cnt[s];
    }
    m.recv_src_off[R] = n_recv;
    for (int q = 0; q < El; ++q) {
      m.recv_expert_off[q] = acc;
      acc += m.recv_expert_cnt[q];
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
    if (host_word) {
      host_word[1] = n_recv;
      __threadfence_system();
      host_word[0] = g.epoch_wait;
    }
  }
}

// Bounded wait for every peer's dispatch flag (R threads of one CTA).
__device__ void dispatch_tail_wait(const EpGeom& g, const EpRegions& rg, char* self_base, int* status) {
  if ((int)threadIdx.x < g.R) {
    const int* flags = reinterpret_cast<const int*>(self_base + rg.flags) + kChDispatch * kMaxRanks;
    wait_flag_ge(flags + threadIdx.x, g.epoch, g.timeout_ns, status, kTimeoutDispatch);
  }
}

template <int MODE, bool FP8, bool CACHED>
__global__ void __launch_bounds__(kSendWarps * 32)
dispatch_send_kernel(EpGeom g, EpRegions rg, PeerPtrs peers, EpMeta m,
                     const char* __restrict__ x, int row_bytes_in,
                     const long long* __restrict__ topk_idx, const float* __restrict__ topk_w,
                     const int* __restrict__ item_rank, const int* __restrict__ chunk_base,
                     int* send_row, int* send_slot, unsigned int* block_counter, int* host_word,
                     int* status, const float* __restrict__ scales_in) {
  extern __shared__ int dyn[];               // [B] send_base, [B] comb_base, [E] scratch
  __shared__ char* s_dst[kSendWarps][kMaxItemsPerToken];
  __shared__ float* s_scl[kSendWarps][kMaxItemsPerToken];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int J = g.J, K = g.K, El = g.El;
  const int row_bytes_out = FP8 ? g.H : row_bytes_in;
  const int scale_cols = g.H / 128;
  const int gw = blockIdx.x * kSendWarps + warp, nw = gridDim.x * kSendWarps;
  char* self_base = peers.base[g.rank];
  int* s_send_base = dyn;
  int* s_comb_base = dyn + g.B;

  int n_tokens = g.T;
  if (!CACHED) {
    // After a notify time-out the prefix tables are not valid: store nothing (the flags below are
    // still raised so that healthy peers are not kept waiting by this rank).
    const bool ok = dispatch_prologue(g, rg, self_base, s_send_base, s_comb_base, dyn + 2 * g.B, status);
    if (blockIdx.x == 0)
      dispatch_publish_meta(g, rg, peers, self_base, m, s_send_base, s_comb_base, host_word, status, ok);
    if (!ok) n_tokens = 0;
  }

  for (int t = gw; t < n_tokens; t += nw) {
    int row = -1, slot = -1, d = 0;
    if (lane < J) {
      long long e = (MODE == 1) ? topk_idx[(size_t)t * K + lane] : 0;
      if (CACHED) {
        row = send_row[(size_t)t * J + lane];
        slot = send_slot[(size_t)t * J + lane];
        // the handle's rows were computed for the capacity of ITS dispatch: never trust them blindly
        if (row >= g.cap || slot >= g.slot_cap) {
          set_status(status, kOverflowRecv);
          row = -1;
          slot = -1;
        }
      } else {
        const int ir = item_rank[(size_t)t * J + lane];
        if (ir >= 0) {
          const int b = (MODE == 0) ? lane : (int)e;
          const int pos = chunk_base[(size_t)(t / kChunkTokens) * g.B + b] + ir;
          row = s_send_base[b] + pos;
          slot = s_comb_base[b] + pos;
          if (row >= g.cap || slot >= g.slot_cap || row < 0 || slot < 0) {
            set_status(status, kOverflowRecv);
            row = -1;
            slot = -1;
          }
        }
        send_row[(size_t)t * J + lane] = row;
        send_slot[(size_t)t * J + lane] = slot;
      }
      d = (MODE == 0) ? lane : (int)(e >= 0 && e < g.E ? e / El : 0);
      if (row >= 0) {
        char* pb = peers.base[d];
        reinterpret_cast<int2*>(pb + rg.recv_meta)[row] = make_int2(slot, g.rank);
        if (MODE == 1)
          reinterpret_cast<float*>(pb + rg.recv_prob)[row] = topk_w ? topk_w[(size_t)t * K + lane] : 1.f;
        s_dst[warp][lane] = pb + rg.recv_x + (size_t)row * row_bytes_out;
        s_scl[warp][lane] = reinterpret_cast<float*>(pb + rg.recv_scales) + (size_t)row * scale_cols;
      }
    }
    const unsigned vmask = __ballot_sync(0xffffffffu, row >= 0);
    __syncwarp();
    if (MODE == 0 && topk_idx != nullptr) {
      // Forward the routing of this token, re-based to the destination's local expert ids.
      const long long my_e = lane < K ? topk_idx[(size_t)t * K + lane] : -1;
      const float my_w = (lane < K && topk_w) ? topk_w[(size_t)t * K + lane] : 0.f;
      for (unsigned mm = vmask; mm; mm &= mm - 1) {
        const int j = __ffs(mm) - 1;
        const int r = __shfl_sync(0xffffffffu, row, j);
        if (lane < K) {
          const long long lo = (long long)j * El;
          const bool mine = my_e >= lo && my_e < lo + El;
          char* pb = peers.base[j];
          reinterpret_cast<long long*>(pb + rg.recv_topk_idx)[(size_t)r * K + lane] = mine ? my_e - lo : -1;
          reinterpret_cast<float*>(pb + rg.recv_topk_w)[(size_t)r * K + lane] = mine ? my_w : 0.f;
        }
      }
    }
    if (vmask == 0) continue;
    const char* src = x + (size_t)t * row_bytes_in;
    if (!FP8) {
      const int nvec = row_bytes_in >> 4;
      for (int v0 = 0; v0 < nvec; v0 += 32 * kUnroll) {
        uint4 buf[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
          const int v = v0 + u * 32 + lane;
          if (v < nvec) buf[u] = ld_global_nc_v4(src + ((size_t)v << 4));
        }
        for (unsigned mm = vmask; mm; mm &= mm - 1) {
          char* dst = s_dst[warp][__ffs(mm) - 1];
#pragma unroll
          for (int u = 0; u < kUnroll; ++u) {
            const int v = v0 + u * 32 + lane;
            if (v < nvec) st_global_v4(dst + ((size_t)v << 4), buf[u]);
          }
        }
      }
      if (scales_in != nullptr) {
        // input was quantised by the caller: its per-128-channel scales travel with the row
        for (int c = lane; c < scale_cols; c += 32) {
          const float sc = scales_in[(size_t)t * scale_cols + c];
          for (unsigned mm = vmask; mm; mm &= mm - 1) s_scl[warp][__ffs(mm) - 1][c] = sc;
        }
      }
    } else {
      // 16 bf16 per lane per step; 8 lanes share one 128-channel scale block.
      const int nsteps = (g.H + 511) / 512;
      for (int it = 0; it < nsteps; ++it) {
        const int el = it * 512 + lane * 16;
        const bool act = el < g.H;
        uint4 a = make_uint4(0, 0, 0, 0), b = a;
        if (act) {
          a = ld_global_nc_v4(src + (size_t)el * 2);
          b = ld_global_nc_v4(src + (size_t)el * 2 + 16);
        }
        float scale;
        const uint4 o = cast_block_fp8(a, b, &scale);
        if (act) {
          for (unsigned mm = vmask; mm; mm &= mm - 1) {
            const int j = __ffs(mm) - 1;
            st_global_v4(s_dst[warp][j] + el, o);
            if ((lane & 7) == 0) s_scl[warp][j][el >> 7] = scale;
          }
        }
      }
    }
    __syncwarp();
  }

  if (last_block_arrive(block_counter, gridDim.x)) {
    if ((int)threadIdx.x < g.R) {
      int* flag = reinterpret_cast<int*>(peers.base[threadIdx.x] + rg.flags) +
                  kChDispatch * kMaxRanks + g.rank;
      st_release_sys(flag, g.epoch);
    }
    if (g.tail_wait) dispatch_tail_wait(g, rg, self_base, status);
  }
}

#define B200EP_LAUNCH_DISPATCH(MODE, FP8, CACHED)                                              \
  dispatch_send_kernel<MODE, FP8, CACHED><<<blocks, kSendWarps * 32, smem, st>>>(              \
      g, rg, peers, m, x, row_bytes_in, topk_idx, topk_w, item_rank, chunk_base, send_row,     \
      send_slot, block_counter, host_word, status, scales_in)

void launch_dispatch_send(const EpGeom& g, const EpRegions& rg, const PeerPtrs& peers,
                          const EpMeta& m, const char* x, int row_bytes_in, bool fp8, bool cached,
                          const long long* topk_idx, const float* topk_w, const int* item_rank,
                          const int* chunk_base, int* send_row, int* send_slot,
                          unsigned int* block_counter, int* host_word, int* status, int blocks,
                          cudaStream_t st, const float* scales_in) {
  if (blocks < 1) blocks = 1;
  const size_t smem = sizeof(int) * (2 * (size_t)g.B + g.E);
  if (g.mode == 0) {
    if (fp8) { if (cached) B200EP_LAUNCH_DISPATCH(0, true, true); else B200EP_LAUNCH_DISPATCH(0, true, false); }
    else     { if (cached) B200EP_LAUNCH_DISPATCH(0, false, true); else B200EP_LAUNCH_DISPATCH(0, false, false); }
  } else {
    if (fp8) { if (cached) B200EP_LAUNCH_DISPATCH(1, true, true); else B200EP_LAUNCH_DISPATCH(1, true, false); }
    else     { if (cached) B200EP_LAUNCH_DISPATCH(1, false, true); else B200EP_LAUNCH_DISPATCH(1, false, false); }
  }
}

}  // namespace b200ep
