// Low-latency (decode) dispatch and combine.
//
// Not exercised by the reference scripts (they only drive DeepEP's normal mode); the call
// shapes follow upstream DeepEP's `low_latency_dispatch` / `low_latency_combine`. Design:
//  * rows land PACKED per local expert, in arrival order: a sender takes the next free row of
//    expert e on the destination with one remote atomic add on that expert's counter and stores
//    the row there (capacity R x M rows per expert, which R senders of at most M tokens cannot
//    exceed). No count exchange, no receiver-side packing copy: the tensors that
//    `low_latency_dispatch` returns ARE the receive region (fixed addresses, usable under graph
//    replay). One copy per (token, expert), fp8 e4m3 with 1x128 scales (or bf16); each row carries
//    (source rank, token, k) so the result can be returned;
//  * the receive region is single-buffered: a rank may dispatch again only after a combine (whose
//    completion proves that every peer has consumed its rows) or a barrier; the host inserts the
//    barrier when two dispatches follow each other;
//  * no host synchronisation and no host-side state per call: the call's epoch lives in device
//    memory and is advanced by the kernel itself, regions are double-buffered by its parity,
//    every kernel argument is constant -> the four kernels can be captured in a CUDA graph;
//  * send and receive halves are separate launches (receive = bounded wait on the peers'
//    flags, then local packing / weighted reduction), which also gives hook-style completion.
#include <cuda_bf16.h>
#include "cast.cuh"
#include "ep.cuh"
#include "ll_api.h"

namespace b200ep {

constexpr int kLLThreads = 256;  // 8 warps work on one row together

// Per-op device state (6 ints): [0] committed epoch, [1] committed arrival target,
// [2] epoch published by the send half, [3] target published by the send half,
// [4] cumulative count of send CTAs that have finished (signal mode 1), [5] unused.
// Send half: works with epoch = [0]+1, target = [1]+grid; CTA 0 publishes them in [2],[3].
// Receive half (next launch on the stream): reads [2],[3]; CTA 0 commits them to [0],[1].
// No kernel ever reads a word that another CTA of the same launch writes.
// The arrival target is a cumulative count modulo 2^32 (it grows by the grid size per call and
// passes 2^31 after a few hours of decode steps): it is advanced in unsigned arithmetic and compared
// with `counter_reached`, never with a signed `>=`. Epochs grow by 1 per call and stay signed.
struct LLTick { int epoch; unsigned int target; };

// First statement of every kernel below. When a kernel is launched with programmatic stream
// serialisation (P.pdl), its CTAs may be placed on the SMs while the previous kernel of the stream
// is still running: `griddepcontrol.wait` holds them until that kernel has completed and its
// writes are visible, so only the launch latency overlaps, never the work. Each kernel at once
// lets ITS successor do the same. Without the launch attribute both instructions do nothing.
__device__ __forceinline__ void ll_stream_order() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ LLTick ll_tick_send(int* st, int grid_ctas) {
  __shared__ int s_e, s_t;
  if (threadIdx.x == 0) {
    s_e = *reinterpret_cast<volatile int*>(st + 0) + 1;
    s_t = (int)((unsigned int)*reinterpret_cast<volatile int*>(st + 1) + (unsigned int)grid_ctas);
    if (blockIdx.x == 0 && blockIdx.y == 0) { st[2] = s_e; st[3] = s_t; }
  }
  __syncthreads();
  return LLTick{s_e, (unsigned int)s_t};
}
__device__ __forceinline__ LLTick ll_tick_recv(int* st) {
  __shared__ int s_e, s_t;
  if (threadIdx.x == 0) {
    s_e = *reinterpret_cast<volatile int*>(st + 2);
    s_t = *reinterpret_cast<volatile int*>(st + 3);
    if (blockIdx.x == 0 && blockIdx.y == 0) { st[0] = s_e; st[1] = s_t; }
  }
  __syncthreads();
  return LLTick{s_e, (unsigned int)s_t};
}
// Every CTA of a send kernel ends with this. A receiver waits for this rank's arrival counter
// (one per peer and channel, cumulative) to reach the target, i.e. for ALL CTAs of the sender
// (the grid size is the same on every rank). Two ways to get there (P.signal_mode):
//  0: every CTA makes its stores visible system-wide and adds 1 to the counter on every peer:
//     no CTA waits for the others, but a receiver takes R x grid remote atomics on R words;
//  1: every CTA makes its stores visible and counts itself on a LOCAL cumulative counter
//     (state[4]); the CTA that completes a multiple of the grid size adds the whole grid size to
//     the counter on every peer: R remote atomics per rank, at the price of one more hop.
// Mode 0 measured faster with 2 ranks, mode 1 with 8.
__device__ __forceinline__ void ll_arrive_on_peers(const LLParams& P, const PeerPtrs& peers, int channel,
                                                   int* state, unsigned int grid_ctas) {
  __shared__ unsigned int s_add;
  __syncthreads();
  if (P.signal_mode == 0) {
    if (threadIdx.x == 0) s_add = 1u;
  } else if (threadIdx.x == 0) {
    fence_acq_rel_sys();
    const unsigned int prev = atomicAdd(reinterpret_cast<unsigned int*>(state + 4), 1u);
    const bool last = ((prev + 1u) % grid_ctas) == 0u;
    // the last CTA acquires what the others published before they counted themselves
    if (last) asm volatile("fence.acq_rel.gpu;" ::: "memory");
    s_add = last ? grid_ctas : 0u;
  }
  __syncthreads();
  const unsigned int add = s_add;
  if (add != 0u && threadIdx.x < P.R) {
    unsigned int* ctr = reinterpret_cast<unsigned int*>(peers.base[threadIdx.x] + P.flags) + channel * kMaxRanks + P.rank;
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(ctr), "r"(add) : "memory");
  }
}

// ---------------------------------------------------------------------------------------
// dispatch, send half: one CTA per token at a time.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kLLThreads)
ll_dispatch_send_kernel(LLParams P, PeerPtrs peers, const char* __restrict__ x,
                        const long long* __restrict__ topk_idx, int* send_cnt_all, int* state,
                        int* status, int* __restrict__ send_slot) {
  __shared__ char* s_dst[kMaxItemsPerToken];
  __shared__ float* s_scl[kMaxItemsPerToken];
  __shared__ int s_n;
  ll_stream_order();
  const LLTick tk = ll_tick_send(state, gridDim.x);
  const int epoch = tk.epoch;
  const int par = epoch & 1;
  (void)send_cnt_all;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = kLLThreads / 32;
  const int row_bytes = P.fp8 ? P.H : P.H * 2;
  const int scale_cols = P.H / 128;
  for (int t = blockIdx.x; t < P.T; t += gridDim.x) {
    if (threadIdx.x == 0) s_n = 0;
    __syncthreads();
    if (threadIdx.x < P.K) {
      const long long e = topk_idx[(size_t)t * P.K + threadIdx.x];
      int given = -1;
      if (e >= 0 && e < P.E) {
        const int d = (int)e / P.El, el = (int)e % P.El;
        char* pb = peers.base[d];
        // next free row of local expert `el` on rank d (rows of one expert are packed in arrival order)
        unsigned int* ctr = reinterpret_cast<unsigned int*>(pb + P.count[par]) + el;
        unsigned int slot;
        asm volatile("atom.add.relaxed.sys.global.u32 %0, [%1], 1;" : "=r"(slot) : "l"(ctr) : "memory");
        if (slot < (unsigned int)(P.R * P.M)) {
          given = (int)slot;
          const size_t row = (size_t)el * P.R * P.M + slot;
          reinterpret_cast<int*>(pb + P.recv_src[0])[row] = (P.rank << 24) | (t << 5) | (int)threadIdx.x;
          const int i = atomicAdd(&s_n, 1);
          s_dst[i] = pb + P.recv_x[0] + row * row_bytes;
          s_scl[i] = reinterpret_cast<float*>(pb + P.recv_scales[0]) + row * scale_cols;
        } else {
          set_status(status, kOverflowRecv);
        }
      } else if (e != -1) {
        set_status(status, kBadExpertIndex);
      }
      if (send_slot != nullptr) send_slot[(size_t)t * P.K + threadIdx.x] = given;
    }
    __syncthreads();
    const int n = s_n;
    const char* src = x + (size_t)t * P.H * 2;
    if (P.fp8) {
      const int nsteps = (P.H + 511) / 512;
      // up to 4 steps per warp with all loads issued before the first conversion
      for (int it0 = warp; it0 < nsteps; it0 += 4 * nwarps) {
        uint4 a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int el = (it0 + u * nwarps) * 512 + lane * 16;
          a[u] = make_uint4(0, 0, 0, 0);
          b[u] = a[u];
          if (it0 + u * nwarps < nsteps && el < P.H) {
            a[u] = ld_global_nc_v4(src + (size_t)el * 2);
            b[u] = ld_global_nc_v4(src + (size_t)el * 2 + 16);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (it0 + u * nwarps >= nsteps) break;       // uniform per warp
          const int el = (it0 + u * nwarps) * 512 + lane * 16;
          float scale;
          const uint4 o = cast_block_fp8(a[u], b[u], &scale);
          if (el < P.H) {
            for (int j = 0; j < n; ++j) {
              st_global_v4(s_dst[j] + el, o);
              if ((lane & 7) == 0) s_scl[j][el >> 7] = scale;
            }
          }
        }
      }
    } else {
      const int nvec = (P.H * 2) >> 4;
      for (int v0 = threadIdx.x; v0 < nvec; v0 += 4 * kLLThreads) {
        uint4 val[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (v0 + u * kLLThreads < nvec) val[u] = ld_global_nc_v4(src + ((size_t)(v0 + u * kLLThreads) << 4));
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (v0 + u * kLLThreads < nvec)
            for (int j = 0; j < n; ++j) st_global_v4(s_dst[j] + ((size_t)(v0 + u * kLLThreads) << 4), val[u]);
      }
    }
    __syncthreads();
  }
  ll_arrive_on_peers(P, peers, kChLLDispatch, state, gridDim.x);
}

// ---------------------------------------------------------------------------------------
// dispatch, receive half: wait for every source's arrival, then read (and clear) the per-expert
// row counters. One CTA; nothing is copied.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kLLThreads)
ll_dispatch_recv_kernel(LLParams P, char* self_base, int* __restrict__ out_count, int* state, int* status) {
  __shared__ int ok;
  ll_stream_order();
  const LLTick tk = ll_tick_recv(state);
  const int par = tk.epoch & 1;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < P.R) {
    const int* flags = reinterpret_cast<const int*>(self_base + P.flags) + kChLLDispatch * kMaxRanks;
    if (!wait_counter_reached(flags + threadIdx.x, tk.target, P.timeout_ns, status, kTimeoutLowLatency)) ok = 0;
  }
  __syncthreads();
  int* cnt = reinterpret_cast<int*>(self_base + P.count[par]);
  for (int el = threadIdx.x; el < P.El; el += kLLThreads) {
    int c = ok ? __ldcg(&cnt[el]) : 0;
    c = c < 0 ? 0 : (c > P.R * P.M ? P.R * P.M : c);
    out_count[el] = c;
    cnt[el] = 0;                 // this parity is used again two dispatches from now
  }
}

// ---------------------------------------------------------------------------------------
// combine, send half: row (el, j) goes back to its source's slot (token, k). grid = (El, split)
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kLLThreads)
ll_combine_send_kernel(LLParams P, PeerPtrs peers, const char* __restrict__ x,
                       const int* __restrict__ src_info, const int* __restrict__ count,
                       int* state, int* status) {
  ll_stream_order();
  const LLTick tk = ll_tick_send(state, gridDim.x * gridDim.y);
  const int par = tk.epoch & 1;
  const int el = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = kLLThreads / 32;
  const size_t cap = (size_t)P.R * P.M;
  int total = __ldcg(&count[el]);
  total = total < 0 ? 0 : (total > (int)cap ? (int)cap : total);
  const int row_bytes = P.H * 2;
  // rows of one expert arrive interleaved from all source ranks: every warp takes a contiguous slice
  const int nslices = gridDim.y * nwarps;
  const int per = (total + nslices - 1) / nslices;
  const int j0 = (blockIdx.y * nwarps + warp) * per;
  const int j1 = min(total, j0 + per);
  for (int j = j0; j < j1; ++j) {
    const int info = __ldcg(&src_info[(size_t)el * cap + j]);
    const int s = (info >> 24) & 0xff, t = (info & 0xffffff) >> 5, k = info & 31;
    if (s >= P.R || t >= P.M || k >= P.K) {
      if (lane == 0) set_status(status, kOverflowSlots);
      continue;
    }
    const char* src = x + ((size_t)el * cap + j) * row_bytes;
    char* dst = peers.base[s] + P.comb_x[par] + ((size_t)t * P.K + k) * row_bytes;
    const int nv = row_bytes >> 4;
    for (int v0 = lane; v0 < nv; v0 += 32 * 14) {
      uint4 buf[14];
#pragma unroll
      for (int u = 0; u < 14; ++u)
        if (v0 + u * 32 < nv) buf[u] = ld_global_nc_v4(src + ((size_t)(v0 + u * 32) << 4));
#pragma unroll
      for (int u = 0; u < 14; ++u)
        if (v0 + u * 32 < nv) st_global_v4(dst + ((size_t)(v0 + u * 32) << 4), buf[u]);
    }
  }
  ll_arrive_on_peers(P, peers, kChLLCombine, state, gridDim.x * gridDim.y);
}

// combine, receive half: out[t] = sum_k w[t,k] * slot(t,k) over k with topk_idx[t,k] >= 0.
__global__ void __launch_bounds__(kLLThreads)
ll_combine_recv_kernel(LLParams P, char* self_base, const long long* __restrict__ topk_idx,
                       const float* __restrict__ topk_w, char* __restrict__ out,
                       int* state, int* status) {
  __shared__ float s_w[kMaxItemsPerToken];
  __shared__ int ok;
  ll_stream_order();
  const LLTick tk = ll_tick_recv(state);
  const int par = tk.epoch & 1;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < P.R) {
    const int* flags = reinterpret_cast<const int*>(self_base + P.flags) + kChLLCombine * kMaxRanks;
    if (!wait_counter_reached(flags + threadIdx.x, tk.target, P.timeout_ns, status, kTimeoutLowLatency)) ok = 0;
  }
  __syncthreads();
  if (!ok) return;
  const int row_bytes = P.H * 2;
  const int nvec = row_bytes >> 4;
  for (int t = blockIdx.x; t < P.T; t += gridDim.x) {
    if (threadIdx.x < P.K) {
      const long long e = topk_idx[(size_t)t * P.K + threadIdx.x];
      s_w[threadIdx.x] = (e >= 0 && e < P.E) ? (topk_w ? topk_w[(size_t)t * P.K + threadIdx.x] : 1.f) : 0.f;
    }
    __syncthreads();
    const char* base = self_base + P.comb_x[par] + (size_t)t * P.K * row_bytes;
    for (int v = threadIdx.x; v < nvec; v += kLLThreads) {
      float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int k0 = 0; k0 < P.K; k0 += 8) {
        uint4 val[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)       // loads first (independent), then the fp32 accumulation
          if (k0 + u < P.K && s_w[k0 + u] != 0.f)
            val[u] = ld_global_v4(base + (size_t)(k0 + u) * row_bytes + ((size_t)v << 4));
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          if (k0 + u >= P.K) break;
          const float w = s_w[k0 + u];
          if (w == 0.f) continue;
          const uint32_t uu[4] = {val[u].x, val[u].y, val[u].z, val[u].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) { a[2 * q] += w * bf16lo(uu[q]); a[2 * q + 1] += w * bf16hi(uu[q]); }
        }
      }
      uint4 o;
      uint32_t* ou = &o.x;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a[2 * q], a[2 * q + 1]);
        ou[q] = *reinterpret_cast<uint32_t*>(&h);
      }
      st_global_v4(out + (size_t)t * row_bytes + ((size_t)v << 4), o);
    }
    __syncthreads();
  }
}


// ---------------------------------------------------------------------------------------
// combine, pull form: announce, wait, load + reduce. One warp per (token, eighth of the row);
// the rows of four experts are requested together, so a token costs two NVLink round trips.
// ---------------------------------------------------------------------------------------
constexpr int kPullGroup = 4;    // contributors whose loads are in flight together
constexpr int kPullUnroll = 4;   // 16-byte vectors per lane and contributor

__global__ void __launch_bounds__(kLLThreads)
ll_combine_pull_kernel(LLParams P, PeerPtrs peers, int phase, const int* __restrict__ send_slot, const long long* __restrict__ topk_idx,
                       const float* __restrict__ topk_w, char* __restrict__ out, int* state, int* status) {
  __shared__ int s_epoch;
  __shared__ unsigned int s_target;
  __shared__ int s_ok;
  ll_stream_order();
  // state: [0] committed epoch, [1] committed arrival target, [2],[3] the pair published by an
  // announce-only launch, [4] CTAs of this launch that have finished
  if (threadIdx.x == 0) {
    if (phase == 2) {
      s_epoch = *reinterpret_cast<volatile int*>(state + 2);
      s_target = (unsigned int)*reinterpret_cast<volatile int*>(state + 3);
    } else {
      s_epoch = *reinterpret_cast<volatile int*>(state + 0) + 1;
      s_target = (unsigned int)*reinterpret_cast<volatile int*>(state + 1) + 1u;
      if (phase == 1) { state[2] = s_epoch; state[3] = (int)s_target; }
    }
    s_ok = 1;
  }
  __syncthreads();
  const int epoch = s_epoch;
  const unsigned int target = s_target;
  char* self_base = peers.base[P.rank];
  if (phase != 2 && blockIdx.x == 0) {
    // announce: my expert output (written by earlier kernels of this stream) may be read
    if ((int)threadIdx.x < P.R) {
      unsigned int* ctr = reinterpret_cast<unsigned int*>(peers.base[threadIdx.x] + P.flags) + kChLLPull * kMaxRanks + P.rank;
      asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(ctr), "r"(1u) : "memory");
    }
  }
  if (phase == 1) return;
  if ((int)threadIdx.x < P.R) {
    const int* flags = reinterpret_cast<const int*>(self_base + P.flags) + kChLLPull * kMaxRanks;
    if (!wait_counter_reached(flags + threadIdx.x, target, P.timeout_ns, status, kTimeoutLowLatency)) s_ok = 0;
  }
  __syncthreads();
  if (s_ok) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = kLLThreads / 32;
    const int row_bytes = P.H * 2;
    const int nvec = row_bytes >> 4;
    int parts = (nvec + 32 * kPullUnroll - 1) / (32 * kPullUnroll);   // one batch of loads per warp and contributor
    if (parts < 1) parts = 1;
    const int part_vec = (nvec + parts - 1) / parts;
    const size_t cap = (size_t)P.R * P.M;
    const int items = P.T * parts;
    for (int it = blockIdx.x * nwarps + warp; it < items; it += gridDim.x * nwarps) {
      const int t = it / parts, part = it % parts;
      const int v_lo = part * part_vec, v_hi = min(nvec, v_lo + part_vec);
      float acc[kPullUnroll][8];
#pragma unroll
      for (int u = 0; u < kPullUnroll; ++u)
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[u][q] = 0.f;
      for (int k0 = 0; k0 < P.K; k0 += kPullGroup) {
        uint4 val[kPullGroup][kPullUnroll];
        float wk[kPullGroup];
#pragma unroll
        for (int g = 0; g < kPullGroup; ++g) {
          const int k = k0 + g;
          wk[g] = 0.f;
          if (k >= P.K) continue;
          const long long e = topk_idx[(size_t)t * P.K + k];
          const int slot = send_slot[(size_t)t * P.K + k];
          if (e < 0 || e >= P.E || slot < 0) continue;
          const int d = (int)e / P.El, el = (int)e % P.El;
          if ((size_t)slot >= cap) continue;
          wk[g] = topk_w ? topk_w[(size_t)t * P.K + k] : 1.f;
          // the row that dispatch stored for (t, k): packed row `slot` of local expert el on rank d
          const char* rowp = peers.base[d] + P.comb_in + ((size_t)el * cap + slot) * row_bytes;
#pragma unroll
          for (int u = 0; u < kPullUnroll; ++u) {
            const int v = v_lo + u * 32 + lane;
            if (v < v_hi) val[g][u] = ld_global_v4(rowp + ((size_t)v << 4));
          }
        }
#pragma unroll
        for (int g = 0; g < kPullGroup; ++g) {
          if (wk[g] == 0.f) continue;
#pragma unroll
          for (int u = 0; u < kPullUnroll; ++u) {
            if (v_lo + u * 32 + lane >= v_hi) continue;
            const uint32_t uu[4] = {val[g][u].x, val[g][u].y, val[g][u].z, val[g][u].w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              acc[u][2 * q] += wk[g] * bf16lo(uu[q]);
              acc[u][2 * q + 1] += wk[g] * bf16hi(uu[q]);
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < kPullUnroll; ++u) {
        const int v = v_lo + u * 32 + lane;
        if (v >= v_hi) continue;
        uint4 o;
        uint32_t* ou = &o.x;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          __nv_bfloat162 h = __floats2bfloat162_rn(acc[u][2 * q], acc[u][2 * q + 1]);
          ou[q] = *reinterpret_cast<uint32_t*>(&h);
        }
        st_global_v4(out + (size_t)t * row_bytes + ((size_t)v << 4), o);
      }
    }
  }
  // the CTA that finishes last commits the epoch (every CTA has read the old one by then)
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(reinterpret_cast<unsigned int*>(state + 4), 1u);
    if (prev == gridDim.x - 1) {
      state[4] = 0;
      state[0] = epoch;
      state[1] = (int)target;
    }
  }
}

// ---- launchers -------------------------------------------------------------------------
// The dispatch send grid is ALWAYS P.G CTAs and the combine send grid ALWAYS (El, P.Gc / El):
// receivers count arrivals, so the number of CTAs must be the same on every rank.
template <typename... KArgs>
static void ll_launch(void (*kern)(KArgs...), dim3 grid, bool pdl, cudaStream_t st, KArgs... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(kLLThreads, 1, 1);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, kern, args...);
}

void launch_ll_dispatch_send(const LLParams& P, const PeerPtrs& peers, const char* x,
                             const long long* topk_idx, int* send_cnt, int* state, int* status,
                             cudaStream_t st, int* send_slot) {
  ll_launch(ll_dispatch_send_kernel, dim3(P.G), P.pdl != 0, st, P, peers, x, topk_idx, send_cnt, state, status,
            send_slot);
}
void launch_ll_dispatch_recv(const LLParams& P, char* self_base, int* out_count, int* state, int* status,
                             cudaStream_t st) {
  ll_launch(ll_dispatch_recv_kernel, dim3(1), P.pdl != 0, st, P, self_base, out_count, state, status);
}
void launch_ll_combine_send(const LLParams& P, const PeerPtrs& peers, const char* x, const int* src_info,
                            const int* count, int* state, int* status, cudaStream_t st) {
  ll_launch(ll_combine_send_kernel, dim3(P.El, P.Gc / P.El), P.pdl != 0, st, P, peers, x, src_info, count, state, status);
}
void launch_ll_combine_recv(const LLParams& P, char* self_base, const long long* topk_idx,
                            const float* topk_w, char* out, int* state, int* status,
                            int blocks, cudaStream_t st) {
  int g = P.T < blocks ? P.T : blocks;
  if (g < 1) g = 1;
  ll_launch(ll_combine_recv_kernel, dim3(g), P.pdl != 0, st, P, self_base, topk_idx, topk_w, out, state, status);
}

void launch_ll_combine_pull(const LLParams& P, const PeerPtrs& peers, int phase, const int* send_slot,
                            const long long* topk_idx, const float* topk_w, char* out, int* state,
                            int* status, cudaStream_t st) {
  ll_launch(ll_combine_pull_kernel, dim3(phase == 1 ? 1 : P.G), P.pdl != 0, st, P, peers, phase, send_slot,
            topk_idx, topk_w, out, state, status);
}

}  // namespace b200ep
