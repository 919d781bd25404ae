// Grouped expert GEMMs on the 5th-generation tensor cores (tcgen05 + TMEM), bf16 -> f32.
//
//   out[r, :] = epilogue( A[r, :] . W[e(r)]^T )    A: [rows, K] rows grouped by local expert,
//                                                  W: [E_local, N_w, K] (K-major, as nn.Linear)
// Replaces the library grouped GEMM / per-expert F.linear loop of the reference
// (`DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:528-541,590-600`) and, through the
// epilogues, the element-wise kernels and the unpermute + combine send that follow them:
//   EPI_PLAIN   : bf16 store.
//   EPI_SWIGLU  : W holds [gate rows | linear rows]; a tile multiplies 128 gate and the matching
//                 128 linear rows, the epilogue writes silu(gate) * linear * prob[r] as bf16.
//   EPI_COMBINE : the fc2 tile rows are stored straight into the combine slot of each token's
//                 SOURCE rank over NVLink (LSU stores from registers via a per-warp staging
//                 line), so no separate unpermute/combine-send kernel runs; the source reduces
//                 its slots on arrival (combine_reduce_kernel).
// Structure: persistent CTAs, one per SM; warp 0 = TMA producer (plain tile loads of this
// GPU's memory; every CTA fetches its own tiles), warp 1 = MMA issuer and TMEM owner,
// warps 2-5 = epilogue. 2 TMEM accumulators (128 lanes x 256 f32 columns each) so the epilogue
// of tile i overlaps the MMAs of tile i+1. Two forms of the same kernel (template CG):
//   CG = 1: one CTA per 128 x 256 tile; 4-stage ring of A 128x64 + B 256x64 (bf16, 128-byte swizzle).
//   CG = 2: a CTA pair (cluster of two SMs, `cta_group::2`) per 256 x 256 tile. Each CTA loads
//           its own 128 rows of A and HALF of the weight tile (128 of the 256 weight rows); the
//           leader CTA issues one MMA that reads both halves from the two CTAs' shared memory and
//           writes 128 accumulator lanes into each CTA's TMEM. A weight tile is thus fetched once
//           per pair and the shared-memory traffic per flop halves for B; 6-stage ring of 32 KiB.
// The tile list is derived on the device from the per-expert row offsets (no host sync).
// Every mbarrier wait is bounded; on a time-out all roles leave their loops, TMEM is freed.
#include <cuda_bf16.h>
#include "tc05.cuh"
#include "tmap.h"
#include "gemm_api.h"

namespace b200ep {

using namespace tc;

constexpr int BM = 128, BN = 256, BK = 64;                    // BM: rows per CTA
constexpr int A_BYTES = BM * BK * 2, B_HALF_BYTES = 128 * BK * 2;
// per-CTA stage: A tile + the part of the weight tile this CTA holds (all of it, or one half)
template <int CG> struct Ring;
template <> struct Ring<1> { static constexpr int STAGES = 4, STAGE_BYTES = A_BYTES + 2 * B_HALF_BYTES; };
template <> struct Ring<2> { static constexpr int STAGES = 6, STAGE_BYTES = A_BYTES + B_HALF_BYTES; };
constexpr int MAX_STAGES = 6;
constexpr int EPI_ROW_BYTES = 128 + 16;                       // 64 bf16 + pad (bank spread)
constexpr int EPI_WARP_BYTES = 32 * EPI_ROW_BYTES;
constexpr int RING_BYTES = 4 * (A_BYTES + 2 * B_HALF_BYTES);
static_assert(Ring<1>::STAGES * Ring<1>::STAGE_BYTES == RING_BYTES && Ring<2>::STAGES * Ring<2>::STAGE_BYTES == RING_BYTES, "");
constexpr int SMEM_BYTES = RING_BYTES + 4 * EPI_WARP_BYTES + 1024 /*align slack*/;
constexpr int GEMM_THREADS = 192;
constexpr int kMaxLocalExperts = 256;

struct Tile { int e, row0, valid_rows, nt; };

// Tile t -> (expert, first row, valid rows, n-tile) as seen by the calling CTA. A tile spans
// TM = 128 * CG rows; CTA `cta_rank` of a pair owns rows [128 * cta_rank, +128) of it (possibly
// none of them valid). Order inside one expert: bands of `gm` m-tiles; inside a band m runs
// fastest, then n, so the tiles in flight at one time cover a band of activation rows times a
// few weight tiles, the band stays in L2 while all weight tiles pass over it, and an expert
// whose activations exceed L2 is not re-read from HBM once per weight tile.
template <int TM>
__device__ __forceinline__ bool decode_tile(int t, const int* s_tile_off, const int* s_row_off, int El,
                                            int n_tiles, int gm, int cta_rank, Tile& out) {
  if (t >= s_tile_off[El]) return false;
  int e = 0;
  while (e + 1 < El && t >= s_tile_off[e + 1]) ++e;
  const int local = t - s_tile_off[e];
  const int rows = s_row_off[e + 1] - s_row_off[e];
  const int m_tiles = (rows + TM - 1) / TM;
  const int per_band = gm * n_tiles;
  const int band = local / per_band;
  const int idx = local - band * per_band;
  const int band_m = min(gm, m_tiles - band * gm);
  const int mt = band * gm + idx % band_m;
  out.e = e;
  out.nt = idx / band_m;
  out.row0 = s_row_off[e] + mt * TM + cta_rank * BM;
  out.valid_rows = max(0, min(BM, rows - mt * TM - cta_rank * BM));
  return true;
}

__device__ __forceinline__ float silu(float v) { return v / (1.f + __expf(-v)); }

// BMN: the weights are stored [E_local, K, N] (N contiguous) instead of [E_local, N, K]; they are
// then read as an N-major operand (64 x 64 boxes, one 128-byte row of 64 outputs per reduction
// index), which is how the data gradients use the forward weights without a transposed copy.
template <int EPI, int CG, bool BMN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ GemmParams p, const __grid_constant__ PeerPtrs peers) {
  constexpr int STAGES = Ring<CG>::STAGES, STAGE_BYTES = Ring<CG>::STAGE_BYTES, TM = BM * CG;
  extern __shared__ unsigned char smem_raw[];
  __shared__ uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ int s_tile_off[kMaxLocalExperts + 1], s_row_off[kMaxLocalExperts + 1];

  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* epi_smem = smem + RING_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort = &s_abort;
  // work unit = CTA (CG 1) or CTA pair (CG 2); in a pair, rank 0 leads: it owns the barriers the
  // MMA thread waits on and issues every MMA; both CTAs load, both run an epilogue on their own TMEM
  const int cta_rank = CG == 2 ? (int)cluster_cta_rank() : 0;
  const bool leader = cta_rank == 0;
  const int unit = CG == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int n_units = CG == 2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int gm = max(1, p.band_rows / TM);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4 * CG); }
    s_abort = 0;
    fence_barrier_init();
    // device-side tile table: rows per expert come from the dispatch metadata
    int acc = 0;
    for (int e = 0; e < p.El; ++e) {
      int r0 = p.expert_off[e], r1 = p.expert_off[e + 1];
      r0 = max(0, min(r0, p.max_rows));
      r1 = max(r0, min(r1, p.max_rows));
      s_row_off[e] = r0;
      s_row_off[e + 1] = r1;
      s_tile_off[e] = acc;
      acc += ((r1 - r0 + TM - 1) / TM) * p.n_tiles;
    }
    s_tile_off[p.El] = acc;
    prefetch_tmap(&map_a);
    prefetch_tmap(&map_b);
  }
  if (warp == 1) {
    if (CG == 2) tmem_alloc_pair(&s_tmem, 512); else tmem_alloc(&s_tmem, 512);
  }
  fence_before_sync();
  __syncthreads();
  __syncwarp();
  if (CG == 2) cluster_sync_all();      // the peer's barriers are initialised before anything arrives on them
  fence_after_sync();
  const uint32_t tmem_base = s_tmem;
  const int k_blocks = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      uint32_t it = 0;
      Tile tl;
      for (int t = unit; decode_tile<TM>(t, s_tile_off, s_row_off, p.El, p.n_tiles, gm, cta_rank, tl) && !*abort; t += n_units) {
        // weight rows of this tile: [gate 128 | linear 128] for swiglu, 256 consecutive rows otherwise;
        // one CTA loads both halves, a pair splits them
        const int b_first = (EPI == EPI_SWIGLU) ? tl.e * p.w_rows + tl.nt * 128 : tl.e * p.w_rows + tl.nt * BN;
        const int b_second = (EPI == EPI_SWIGLU) ? b_first + p.N : b_first + 128;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (it >= STAGES && !mbar_wait(&empty_bar[s], ph ^ 1, p.status, abort)) break;
          unsigned char* st = smem + s * STAGE_BYTES;
          if (BMN) {
            // weights [K, N] per expert: boxes of 64 reduction rows x 64 output columns. A reduction
            // tail that runs into the next expert's rows meets zero-filled columns of A.
            constexpr int NBOX = CG == 1 ? 4 : 2;
            const int n0 = tl.nt * BN + (CG == 2 ? cta_rank * 128 : 0);
            const int krow = tl.e * p.w_rows + kb * BK;
            if (CG == 1) {
              mbar_expect_tx(&full_bar[s], STAGE_BYTES);
              tma_load_2d(st, &map_a, kb * BK, tl.row0, &full_bar[s]);
#pragma unroll
              for (int b = 0; b < NBOX; ++b) tma_load_2d(st + A_BYTES + b * 8192, &map_b, n0 + b * 64, krow, &full_bar[s]);
            } else {
              if (leader) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
              tma_load_2d_pair(st, &map_a, kb * BK, tl.row0, &full_bar[s]);
#pragma unroll
              for (int b = 0; b < NBOX; ++b) tma_load_2d_pair(st + A_BYTES + b * 8192, &map_b, n0 + b * 64, krow, &full_bar[s]);
            }
          } else if (CG == 1) {
            mbar_expect_tx(&full_bar[s], STAGE_BYTES);
            tma_load_2d(st, &map_a, kb * BK, tl.row0, &full_bar[s]);
            tma_load_2d(st + A_BYTES, &map_b, kb * BK, b_first, &full_bar[s]);
            tma_load_2d(st + A_BYTES + B_HALF_BYTES, &map_b, kb * BK, b_second, &full_bar[s]);
          } else {
            // both CTAs' bytes are counted on the leader's barrier; only the leader announces them
            if (leader) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
            tma_load_2d_pair(st, &map_a, kb * BK, tl.row0, &full_bar[s]);
            tma_load_2d_pair(st + A_BYTES, &map_b, kb * BK, leader ? b_first : b_second, &full_bar[s]);
          }
        }
      }
      if (*abort) {
        // let the loads that are still in flight land before the CTA's shared memory goes away
        // (a pair's follower cannot observe its own loads: they complete on the leader's barrier)
        if (CG == 1 || leader) {
          int quiet = 0;
          for (uint32_t n = it > STAGES ? it - STAGES : 0; n < it; ++n)
            mbar_wait(&full_bar[n % STAGES], (n / STAGES) & 1, nullptr, &quiet);
        }
      } else if (CG == 2) {
        // a pair's CTA must not leave while the leader's last commits can still arrive on its barriers
        for (uint32_t n = it > STAGES ? it - STAGES : 0; n < it; ++n)
          if (!mbar_wait(&empty_bar[n % STAGES], (n / STAGES) & 1, p.status, abort)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (the leader CTA of a pair) ----------------
    if (leader && elect_one()) {
      const uint32_t idesc = instr_desc_bf16(TM, BN, false, BMN);
      uint32_t it = 0, tile_n = 0;
      Tile tl;
      for (int t = unit; decode_tile<TM>(t, s_tile_off, s_row_off, p.El, p.n_tiles, gm, cta_rank, tl) && !*abort; t += n_units, ++tile_n) {
        const int buf = tile_n & 1;
        const uint32_t use = tile_n >> 1;
        if (use > 0 && !mbar_wait(&acc_empty[buf], (use - 1) & 1, p.status, abort)) break;
        fence_after_sync();
        const uint32_t d_tmem = tmem_base + buf * BN;
        bool ok = true;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, p.status, abort)) { ok = false; break; }
          fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t a_desc = smem_desc_sw128(a_addr);
          const uint64_t b_desc = BMN ? smem_desc_mn_sw128(a_addr + A_BYTES, 8192) : smem_desc_sw128(a_addr + A_BYTES);
          // per MMA step of 16 reduction indices: K-major +32 bytes (2 units), N-major +16 rows of 128 bytes (128 units)
          constexpr int B_STEP = BMN ? 128 : 2;
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            if (CG == 1) mma_bf16(d_tmem, a_desc + 2 * k, b_desc + B_STEP * k, idesc, (kb | k) ? 1u : 0u);
            else mma_bf16_pair(d_tmem, a_desc + 2 * k, b_desc + B_STEP * k, idesc, (kb | k) ? 1u : 0u);
          }
          // frees the smem stage (in both CTAs of a pair) when these MMAs retire
          if (CG == 1) mma_commit(&empty_bar[s]); else mma_commit_pair(&empty_bar[s]);
        }
        if (!ok) break;
        // accumulator complete (announced to both epilogues of a pair)
        if (CG == 1) mma_commit(&acc_full[buf]); else mma_commit_pair(&acc_full[buf]);
      }
    }
  } else {
    // ---------------- epilogue (4 warps, one TMEM lane quarter each) ----------------
    const int q = warp & 3;                        // TMEM lanes [32q, 32q+32)
    unsigned char* my_smem = epi_smem + (warp - 2) * EPI_WARP_BYTES;
    uint32_t tile_n = 0;
    Tile tl;
    for (int t = unit; decode_tile<TM>(t, s_tile_off, s_row_off, p.El, p.n_tiles, gm, cta_rank, tl) && !*abort; t += n_units, ++tile_n) {
      const int buf = tile_n & 1;
      if (!mbar_wait(&acc_full[buf], (tile_n >> 1) & 1, p.status, abort)) break;
      fence_after_sync();
      const uint32_t t_addr = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
      const int my_row = tl.row0 + q * 32 + lane;               // the row whose accumulators I load
      const bool row_ok = q * 32 + lane < tl.valid_rows;
      float prob = 1.f;
      if (EPI == EPI_SWIGLU && row_ok && p.row_prob) prob = p.row_prob[my_row];
      constexpr int OUT_COLS = (EPI == EPI_SWIGLU) ? 128 : BN;
      const int col_base = tl.nt * OUT_COLS;
      for (int c = 0; c < OUT_COLS / 64 && tl.valid_rows > 0; ++c) {
        // ---- 64 output columns of my row -> registers -> bf16 -> my row of the staging tile
        uint32_t packed[32];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t v[32];
          tmem_ld32(t_addr + c * 64 + h * 32, v);
          if (EPI == EPI_SWIGLU) {
            uint32_t u[32];
            tmem_ld32(t_addr + 128 + c * 64 + h * 32, u);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float a0 = silu(__uint_as_float(v[2 * i])) * __uint_as_float(u[2 * i]) * prob;
              const float a1 = silu(__uint_as_float(v[2 * i + 1])) * __uint_as_float(u[2 * i + 1]) * prob;
              __nv_bfloat162 hh = __floats2bfloat162_rn(a0, a1);
              packed[h * 16 + i] = *reinterpret_cast<uint32_t*>(&hh);
            }
          } else {
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
              packed[h * 16 + i] = *reinterpret_cast<uint32_t*>(&hh);
            }
          }
        }
        uint4* srow = reinterpret_cast<uint4*>(my_smem + lane * EPI_ROW_BYTES);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          srow[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
        __syncwarp();
        // ---- coalesced: 8 lanes write one row's 128 bytes, 4 rows per step
        const int col0 = col_base + c * 64;
#pragma unroll
        for (int step = 0; step < 8; ++step) {
          const int r = step * 4 + (lane >> 3);
          const int seg = lane & 7;
          const int grow = tl.row0 + q * 32 + r;
          const bool ok = (q * 32 + r) < tl.valid_rows && (col0 + seg * 8) < p.N_out;
          if (ok) {
            const uint4 val = *reinterpret_cast<const uint4*>(my_smem + r * EPI_ROW_BYTES + seg * 16);
            char* dst;
            if (EPI == EPI_COMBINE) {
              const int2 meta = p.recv_meta[grow];
              const bool good = meta.y >= 0 && meta.y < p.R && meta.x >= 0 && meta.x < p.slot_cap;
              dst = good ? peers.base[meta.y] + p.comb_off + ((size_t)meta.x * p.N_out + col0 + seg * 8) * 2 : nullptr;
              if (!good) set_status(p.status, kOverflowSlots);
            } else {
              dst = reinterpret_cast<char*>(p.out) + ((size_t)grow * p.out_ld + col0 + seg * 8) * 2;
            }
            if (dst) st_global_v4(dst, val);
          }
        }
        __syncwarp();
        if (EPI == EPI_SWIGLU && p.pre_out != nullptr) {
          // training forward: also keep the pre-activation [gate | linear] (bf16) for the backward pass
#pragma unroll 1
          for (int half = 0; half < 2; ++half) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t v[32];
              tmem_ld32(t_addr + half * 128 + c * 64 + h * 32, v);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 16; ++i) {
                __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
                packed[h * 16 + i] = *reinterpret_cast<uint32_t*>(&hh);
              }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i)
              srow[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
            __syncwarp();
#pragma unroll
            for (int step = 0; step < 8; ++step) {
              const int r = step * 4 + (lane >> 3);
              const int seg = lane & 7;
              if ((q * 32 + r) < tl.valid_rows && (col0 + seg * 8) < p.N_out) {
                const uint4 val = *reinterpret_cast<const uint4*>(my_smem + r * EPI_ROW_BYTES + seg * 16);
                char* dst = reinterpret_cast<char*>(p.pre_out) +
                            ((size_t)(tl.row0 + q * 32 + r) * p.pre_ld + (size_t)half * p.N + col0 + seg * 8) * 2;
                st_global_v4(dst, val);
              }
            }
            __syncwarp();
          }
        }
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (CG == 1) mbar_arrive(&acc_empty[buf]); else mbar_arrive_cluster(&acc_empty[buf], 0);
      }
    }
  }

  // ---------------- teardown: every path arrives here ----------------
  fence_before_sync();
  __syncthreads();
  __syncwarp();
  if (CG == 2) cluster_sync_all();      // both epilogues are done with TMEM, nobody addresses the peer any more
  if (warp == 1) {
    fence_after_sync();
    if (CG == 2) tmem_dealloc_pair(tmem_base, 512); else tmem_dealloc(tmem_base, 512);
  }
  if (EPI == EPI_COMBINE && p.signal_flag_off >= 0) {
    // all CTAs' peer stores done -> the last CTA raises this rank's combine flag on every peer
    if (last_block_arrive(p.block_counter, gridDim.x)) {
      if (threadIdx.x < p.R) {
        int* flag = reinterpret_cast<int*>(peers.base[threadIdx.x] + p.signal_flag_off) + p.rank;
        st_release_sys(flag, p.epoch);
      }
    }
  }
}

// ---- host side -----------------------------------------------------------------------------
// operand maps: box = 64 columns (one 128-byte swizzle row) x 128 rows
static int make_map(CUtensorMap* m, const void* base, long long rows, long long cols) {
  return make_tmap_bf16(m, base, rows, cols, BK, 128);
}

// Number of CTA pairs that can be resident at once (the SMs of a pair share a GPC, so this can be
// below SMs / 2); cached per epilogue. 0 if the query fails.
template <int EPI, bool BMN>
static int max_resident_pairs() {
  static int cached = -1;
  if (cached < 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, grouped_gemm_kernel<EPI, 2, BMN>, &cfg) != cudaSuccess) n = 0;
    cached = n;
  }
  return cached;
}

template <int EPI, bool BMN>
static int launch_one(const CUtensorMap& ma, const CUtensorMap& mb, const GemmParams& p, const PeerPtrs& peers,
                      int ctas, bool pair, cudaStream_t st) {
  if (!pair) {
    if (cudaFuncSetAttribute(grouped_gemm_kernel<EPI, 1, BMN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return 4;
    grouped_gemm_kernel<EPI, 1, BMN><<<ctas, GEMM_THREADS, SMEM_BYTES, st>>>(ma, mb, p, peers);
    return 0;
  }
  if (cudaFuncSetAttribute(grouped_gemm_kernel<EPI, 2, BMN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
    return 4;
  int pairs = ctas / 2;
  const int resident = max_resident_pairs<EPI, BMN>();
  if (resident < 1) return 5;
  if (pairs > resident) pairs = resident;
  if (pairs < 1) pairs = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<EPI, 2, BMN>, ma, mb, p, peers) == cudaSuccess ? 0 : 5;
}

int launch_grouped_gemm(const void* a, long long a_rows, const void* w, int epi, GemmParams p,
                        const PeerPtrs& peers, int ctas, bool pair, cudaStream_t st) {
  if (p.El < 1 || p.El > kMaxLocalExperts || p.K <= 0 || p.K % 8 || p.N <= 0 || p.N_out % 8) return 1;
  if (reinterpret_cast<uintptr_t>(a) % 16 || reinterpret_cast<uintptr_t>(w) % 16) return 1;
  if (epi == EPI_SWIGLU && (p.N % 128)) return 1;
  CUtensorMap ma, mb;
  if (make_map(&ma, a, a_rows, p.K)) return 3;
  if (p.b_mn) {
    if (epi != EPI_PLAIN) return 1;
    if (make_tmap_bf16(&mb, w, (long long)p.El * p.w_rows, p.N, 64, BK)) return 3;
  } else if (make_map(&mb, w, (long long)p.El * p.w_rows, p.K)) return 3;
  p.n_tiles = epi == EPI_SWIGLU ? p.N / 128 : (p.N + BN - 1) / BN;
  p.max_rows = (int)a_rows;
  if (p.band_rows <= 0) p.band_rows = 2048;
  if (ctas < 1) ctas = 1;
  if (epi == EPI_PLAIN && p.b_mn) return launch_one<EPI_PLAIN, true>(ma, mb, p, peers, ctas, pair, st);
  if (epi == EPI_PLAIN) return launch_one<EPI_PLAIN, false>(ma, mb, p, peers, ctas, pair, st);
  if (epi == EPI_SWIGLU) return launch_one<EPI_SWIGLU, false>(ma, mb, p, peers, ctas, pair, st);
  if (epi == EPI_COMBINE) return launch_one<EPI_COMBINE, false>(ma, mb, p, peers, ctas, pair, st);
  return 1;
}

}  // namespace b200ep
