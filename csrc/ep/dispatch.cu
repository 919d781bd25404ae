// Normal-mode dispatch: ONE kernel reads each local token once, optionally casts it to
// block-scaled fp8 (e4m3, one f32 scale per 128 channels), and stores it straight into its
// final row of every destination rank's receive region over NVLink with 16-byte LSU peer
// stores. The permute is part of the address computation, so no separate permute kernel and
// no staging ring exist. Replaces `Buffer.dispatch` as consumed by
// `DeepEP_v1/deepep_v1_dispatch.py:212-230` and, in expert mode, also the multihot/permute
// glue of `DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:276-388`.
#include <cuda_bf16.h>
#include "cast.cuh"
#include "ep.cuh"
#include "api.h"

namespace b200ep {

constexpr int kSendWarps = 16;  // warps per CTA in the send kernels
constexpr int kUnroll = 4;

template <int MODE, bool FP8, bool CACHED>
__global__ void __launch_bounds__(kSendWarps * 32)
dispatch_send_kernel(EpGeom g, EpRegions rg, PeerPtrs peers, EpMeta m,
                     const char* __restrict__ x, int row_bytes_in,
                     const long long* __restrict__ topk_idx, const float* __restrict__ topk_w,
                     const int* __restrict__ item_rank, const int* __restrict__ chunk_base,
                     int* send_row, int* send_slot, unsigned int* block_counter, int* status,
                     const float* __restrict__ scales_in) {
  __shared__ char* s_dst[kSendWarps][kMaxItemsPerToken];
  __shared__ float* s_scl[kSendWarps][kMaxItemsPerToken];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int J = g.J, K = g.K, El = g.El;
  const int row_bytes_out = FP8 ? g.H : row_bytes_in;
  const int scale_cols = g.H / 128;
  const int gw = blockIdx.x * kSendWarps + warp, nw = gridDim.x * kSendWarps;
  // After a notify time-out the prefix tables are not valid: store nothing (the flags below are
  // still raised so that healthy peers are not kept waiting by this rank).
  const int n_tokens = (!CACHED && *m.send_total < 0) ? 0 : g.T;

  for (int t = gw; t < n_tokens; t += nw) {
    int row = -1, slot = -1, d = 0;
    if (lane < J) {
      long long e = (MODE == 1) ? topk_idx[(size_t)t * K + lane] : 0;
      if (CACHED) {
        row = send_row[(size_t)t * J + lane];
        slot = send_slot[(size_t)t * J + lane];
      } else {
        const int ir = item_rank[(size_t)t * J + lane];
        if (ir >= 0) {
          const int b = (MODE == 0) ? lane : (int)e;
          const int pos = chunk_base[(size_t)(t / kChunkTokens) * g.B + b] + ir;
          row = m.send_base[b] + pos;
          slot = m.comb_base[b] + pos;
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
    if (threadIdx.x < g.R) {
      int* flag = reinterpret_cast<int*>(peers.base[threadIdx.x] + rg.flags) +
                  kChDispatch * kMaxRanks + g.rank;
      st_release_sys(flag, g.epoch);
    }
  }
}

#define B200EP_LAUNCH_DISPATCH(MODE, FP8, CACHED)                                              \
  dispatch_send_kernel<MODE, FP8, CACHED><<<blocks, kSendWarps * 32, 0, st>>>(                 \
      g, rg, peers, m, x, row_bytes_in, topk_idx, topk_w, item_rank, chunk_base, send_row,     \
      send_slot, block_counter, status, scales_in)

void launch_dispatch_send(const EpGeom& g, const EpRegions& rg, const PeerPtrs& peers,
                          const EpMeta& m, const char* x, int row_bytes_in, bool fp8, bool cached,
                          const long long* topk_idx, const float* topk_w, const int* item_rank,
                          const int* chunk_base, int* send_row, int* send_slot,
                          unsigned int* block_counter, int* status, int blocks, cudaStream_t st,
                          const float* scales_in) {
  if (blocks < 1) blocks = 1;
  if (g.mode == 0) {
    if (fp8) { if (cached) B200EP_LAUNCH_DISPATCH(0, true, true); else B200EP_LAUNCH_DISPATCH(0, true, false); }
    else     { if (cached) B200EP_LAUNCH_DISPATCH(0, false, true); else B200EP_LAUNCH_DISPATCH(0, false, false); }
  } else {
    if (fp8) { if (cached) B200EP_LAUNCH_DISPATCH(1, true, true); else B200EP_LAUNCH_DISPATCH(1, true, false); }
    else     { if (cached) B200EP_LAUNCH_DISPATCH(1, false, true); else B200EP_LAUNCH_DISPATCH(1, false, false); }
  }
}

}  // namespace b200ep
