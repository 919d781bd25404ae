// Weight gradients of the grouped expert GEMMs on the 5th-generation tensor cores:
//
//   dW[e] = G_e^T . X_e        G: [rows, M] (gradient w.r.t. the layer's output, rows grouped by
//                              local expert), X: [rows, N] (the layer's input), dW: [E_local, M, N]
//
// i.e. a GEMM whose reduction runs over the RAGGED token dimension of each expert. The reference
// defines this step only through autograd of its per-expert `F.linear` loop
// (`DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:590-600`, never run there).
// Both operands are read as stored (token-major): for the tensor core they are "M/N-major"
// tiles, one 128-byte row of 64 features per token, which is exactly what a TMA box of
// 64 columns x 64 rows with 128-byte swizzle produces, so no transposed copy is made.
// Structure as in grouped_gemm.cu (persistent CTAs, warp 0 TMA producer, warp 1 MMA issuer and
// TMEM owner, warps 2-5 epilogue, two TMEM accumulators, bounded waits, template CG: one CTA
// per 128 x 256 tile of dW, or a CTA pair (`cta_group::2`) per 256 x 256 tile with each CTA
// loading 128 columns of G and 128 of the 256 columns of X).
// Ragged reduction: an expert's rows [r0, r1) are walked in blocks of 64. The rows of the LAST
// block that lie beyond r1 belong to the next expert (or are uninitialised), so the MMA warp
// (all 32 lanes; in a pair the same warp of BOTH CTAs, each for its own shared memory) overwrites
// them with zeros once the block has landed (a whole 128-byte row is swizzle-invariant), fences,
// and only then is the block multiplied. An expert without rows gets a zero gradient.
#include <cuda_bf16.h>
#include "tc05.cuh"
#include "tmap.h"
#include "gemm_api.h"

namespace b200ep {

using namespace tc;

namespace wg {

constexpr int BM = 128, BN = 256, BK = 64;          // BM: dW rows per CTA; BK: tokens per block
constexpr int BOX_BYTES = BK * 128;                  // 64 tokens x 64 features (bf16)
template <int CG> struct Ring;
template <> struct Ring<1> { static constexpr int STAGES = 4, B_BOXES = 4; };   // all 256 X columns
template <> struct Ring<2> { static constexpr int STAGES = 6, B_BOXES = 2; };   // my half of them
constexpr int A_BOXES = BM / 64;
constexpr int MAX_STAGES = 6;
constexpr int RING_BYTES = 4 * (2 + 4) * BOX_BYTES;
constexpr int EPI_ROW_BYTES = 128 + 16;
constexpr int EPI_WARP_BYTES = 32 * EPI_ROW_BYTES;
constexpr int SMEM_BYTES = RING_BYTES + 4 * EPI_WARP_BYTES + 1024;
constexpr int THREADS = 192;
constexpr int kMaxLocalExperts = 256;
constexpr int BAND_M_TILES_ROWS = 2048;              // dW rows per band of the tile order

struct Tile { int e, mt, nt, r0, rows; };

// Tile t -> (expert, m-tile, n-tile, first token row, token rows). Every expert has the same
// m_tiles x n_tiles grid; inside an expert m runs fastest within bands of `gm` m-tiles, then n,
// so the CTAs running together share columns of G and X while they stream over the tokens.
__device__ __forceinline__ bool decode(int t, int El, int m_tiles, int n_tiles, int gm, const int* s_row_off, Tile& o) {
  const int per_e = m_tiles * n_tiles;
  if (t >= El * per_e) return false;
  const int e = t / per_e, local = t - e * per_e;
  const int per_band = gm * n_tiles;
  const int band = local / per_band, idx = local - band * per_band;
  const int band_m = min(gm, m_tiles - band * gm);
  o.e = e;
  o.mt = band * gm + idx % band_m;
  o.nt = idx / band_m;
  o.r0 = s_row_off[e];
  o.rows = s_row_off[e + 1] - s_row_off[e];
  return true;
}

template <int CG>
__global__ void __launch_bounds__(THREADS, 1)
grouped_wgrad_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_x,
                     const __grid_constant__ WgradParams p) {
  constexpr int STAGES = Ring<CG>::STAGES, B_BOXES = Ring<CG>::B_BOXES;
  constexpr int STAGE_BYTES = (A_BOXES + B_BOXES) * BOX_BYTES, TM = BM * CG;
  static_assert(STAGES * STAGE_BYTES == RING_BYTES, "");
  extern __shared__ unsigned char smem_raw[];
  // full_bar: operand bytes landed (pair: counted on the leader, except a follower's tail block,
  // which is counted on the follower's tail_full of that stage); tail_bar (leader): the follower
  // has patched its half of a tail block
  __shared__ uint64_t full_bar[MAX_STAGES], empty_bar[MAX_STAGES], tail_full[MAX_STAGES], acc_full[2], acc_empty[2], tail_bar;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ int s_row_off[kMaxLocalExperts + 1];

  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* epi_smem = smem + RING_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort = &s_abort;
  const int cta_rank = CG == 2 ? (int)cluster_cta_rank() : 0;
  const bool leader = cta_rank == 0;
  const int unit = CG == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int n_units = CG == 2 ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int m_tiles = (p.M + TM - 1) / TM, n_tiles = (p.N + BN - 1) / BN;   // a last m-tile may hang over M: its G columns read as zeros, its dW rows are not stored
  const int gm = max(1, BAND_M_TILES_ROWS / TM);

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); mbar_init(&tail_full[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4 * CG); }
    mbar_init(&tail_bar, 1);
    s_abort = 0;
    fence_barrier_init();
    for (int e = 0; e <= p.El; ++e) {
      int r = p.expert_off[e];
      r = max(0, min(r, p.max_rows));
      if (e > 0) r = max(r, s_row_off[e - 1]);
      s_row_off[e] = r;
    }
    prefetch_tmap(&map_g);
    prefetch_tmap(&map_x);
  }
  if (warp == 1) {
    if (CG == 2) tmem_alloc_pair(&s_tmem, 512); else tmem_alloc(&s_tmem, 512);
  }
  fence_before_sync();
  __syncthreads();
  __syncwarp();
  if (CG == 2) cluster_sync_all();
  fence_after_sync();
  const uint32_t tmem_base = s_tmem;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      uint32_t it = 0;
      Tile tl;
      for (int t = unit; decode(t, p.El, m_tiles, n_tiles, gm, s_row_off, tl) && !*abort; t += n_units) {
        const int k_blocks = (tl.rows + BK - 1) / BK;
        const int a_col = tl.mt * TM + cta_rank * BM;
        const int b_col = tl.nt * BN + (CG == 2 ? cta_rank * 128 : 0);
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (it >= STAGES && !mbar_wait(&empty_bar[s], ph ^ 1, p.status, abort)) break;
          unsigned char* st = smem + s * STAGE_BYTES;
          const int row = tl.r0 + kb * BK;
          const bool tail = (kb == k_blocks - 1) && (tl.rows % BK);
          if (CG == 1) {
            mbar_expect_tx(&full_bar[s], STAGE_BYTES);
#pragma unroll
            for (int b = 0; b < A_BOXES; ++b) tma_load_2d(st + b * BOX_BYTES, &map_g, a_col + b * 64, row, &full_bar[s]);
#pragma unroll
            for (int b = 0; b < B_BOXES; ++b)
              tma_load_2d(st + (A_BOXES + b) * BOX_BYTES, &map_x, b_col + b * 64, row, &full_bar[s]);
          } else if (tail && !leader) {
            // my own warp 1 must see these bytes land before it patches them: count them here
            mbar_expect_tx(&tail_full[s], STAGE_BYTES);
#pragma unroll
            for (int b = 0; b < A_BOXES; ++b) tma_load_2d(st + b * BOX_BYTES, &map_g, a_col + b * 64, row, &tail_full[s]);
#pragma unroll
            for (int b = 0; b < B_BOXES; ++b)
              tma_load_2d(st + (A_BOXES + b) * BOX_BYTES, &map_x, b_col + b * 64, row, &tail_full[s]);
          } else {
            if (leader) mbar_expect_tx(&full_bar[s], tail ? STAGE_BYTES : 2 * STAGE_BYTES);
#pragma unroll
            for (int b = 0; b < A_BOXES; ++b) tma_load_2d_pair(st + b * BOX_BYTES, &map_g, a_col + b * 64, row, &full_bar[s]);
#pragma unroll
            for (int b = 0; b < B_BOXES; ++b)
              tma_load_2d_pair(st + (A_BOXES + b) * BOX_BYTES, &map_x, b_col + b * 64, row, &full_bar[s]);
          }
        }
      }
      if (*abort) {
        if (CG == 1 || leader) {
          int quiet = 0;
          for (uint32_t n = it > STAGES ? it - STAGES : 0; n < it; ++n)
            mbar_wait(&full_bar[n % STAGES], (n / STAGES) & 1, nullptr, &quiet);
        }
      } else if (CG == 2) {
        for (uint32_t n = it > STAGES ? it - STAGES : 0; n < it; ++n)
          if (!mbar_wait(&empty_bar[n % STAGES], (n / STAGES) & 1, p.status, abort)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA warp: all lanes patch tail blocks, one elected lane of the leader issues ----------------
    const bool issuer = elect_one() && leader;
    const uint32_t idesc = instr_desc_bf16(TM, BN, true, true);
    uint32_t it = 0, tile_n = 0, tails = 0, tail_par = 0;
    Tile tl;
    for (int t = unit; decode(t, p.El, m_tiles, n_tiles, gm, s_row_off, tl) && !*abort; t += n_units, ++tile_n) {
      const int k_blocks = (tl.rows + BK - 1) / BK;
      const int valid = tl.rows % BK;
      const int buf = tile_n & 1;
      const uint32_t use = tile_n >> 1;
      if (leader) {
        if (use > 0 && !mbar_wait(&acc_empty[buf], (use - 1) & 1, p.status, abort)) break;
        fence_after_sync();
      }
      const uint32_t d_tmem = tmem_base + buf * BN;
      bool ok = true;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        const bool tail = (kb == k_blocks - 1) && valid;
        if (!leader && !tail) continue;                          // a follower only patches its tail blocks
        if (leader) {
          if (!mbar_wait(&full_bar[s], ph, p.status, abort)) { ok = false; break; }
        } else {
          if (!mbar_wait(&tail_full[s], (tail_par >> s) & 1, p.status, abort)) { ok = false; break; }
          tail_par ^= 1u << s;
        }
        if (tail) {
          unsigned char* st = smem + s * STAGE_BYTES;
          const int per_box = (BK - valid) * 8;                  // 16-byte chunks to clear per box
          for (int i = lane; i < (A_BOXES + B_BOXES) * per_box; i += 32) {
            const int box = i / per_box, rem = i - box * per_box;
            *reinterpret_cast<uint4*>(st + box * BOX_BYTES + (valid + (rem >> 3)) * 128 + (rem & 7) * 16) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (CG == 2) {
            if (!leader) {
              if (lane == 0) mbar_arrive_cluster(&tail_bar, 0);
              continue;
            }
            if (!mbar_wait(&tail_bar, tails & 1, p.status, abort)) { ok = false; break; }
            ++tails;
          }
        }
        fence_after_sync();
        if (issuer) {
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t a_desc = smem_desc_mn_sw128(a_addr, BOX_BYTES);
          const uint64_t b_desc = smem_desc_mn_sw128(a_addr + A_BOXES * BOX_BYTES, BOX_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {  // 16 tokens = 16 rows of 128 bytes: +2048 bytes = +128 units
            if (CG == 1) mma_bf16(d_tmem, a_desc + 128 * k, b_desc + 128 * k, idesc, (kb | k) ? 1u : 0u);
            else mma_bf16_pair(d_tmem, a_desc + 128 * k, b_desc + 128 * k, idesc, (kb | k) ? 1u : 0u);
          }
          if (CG == 1) mma_commit(&empty_bar[s]); else mma_commit_pair(&empty_bar[s]);
        }
        __syncwarp();
      }
      if (!ok) break;
      if (issuer) {
        if (CG == 1) mma_commit(&acc_full[buf]); else mma_commit_pair(&acc_full[buf]);
      }
      __syncwarp();
    }
  } else {
    // ---------------- epilogue (4 warps, one TMEM lane quarter each) ----------------
    const int q = warp & 3;
    unsigned char* my_smem = epi_smem + (warp - 2) * EPI_WARP_BYTES;
    uint32_t tile_n = 0;
    Tile tl;
    for (int t = unit; decode(t, p.El, m_tiles, n_tiles, gm, s_row_off, tl) && !*abort; t += n_units, ++tile_n) {
      const int k_blocks = (tl.rows + BK - 1) / BK;
      const int buf = tile_n & 1;
      if (!mbar_wait(&acc_full[buf], (tile_n >> 1) & 1, p.status, abort)) break;
      fence_after_sync();
      const uint32_t t_addr = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
      const int row_base = tl.mt * TM + cta_rank * BM + q * 32;   // dW row of my warp's first lane
      __nv_bfloat16* out_e = reinterpret_cast<__nv_bfloat16*>(p.out) + (size_t)tl.e * p.M * p.N;
      for (int c = 0; c < BN / 64; ++c) {
        uint32_t packed[32];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t v[32];
          if (k_blocks > 0) {
            tmem_ld32(t_addr + c * 64 + h * 32, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = 0;             // an expert without rows: zero gradient
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            packed[h * 16 + i] = *reinterpret_cast<uint32_t*>(&hh);
          }
        }
        uint4* srow = reinterpret_cast<uint4*>(my_smem + lane * EPI_ROW_BYTES);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          srow[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
        __syncwarp();
        const int col0 = tl.nt * BN + c * 64;
#pragma unroll
        for (int step = 0; step < 8; ++step) {
          const int r = step * 4 + (lane >> 3);
          const int seg = lane & 7;
          if (col0 + seg * 8 < p.N && row_base + r < p.M) {
            const uint4 val = *reinterpret_cast<const uint4*>(my_smem + r * EPI_ROW_BYTES + seg * 16);
            st_global_v4(reinterpret_cast<char*>(out_e + (size_t)(row_base + r) * p.N + col0 + seg * 8), val);
          }
        }
        __syncwarp();
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (CG == 1) mbar_arrive(&acc_empty[buf]); else mbar_arrive_cluster(&acc_empty[buf], 0);
      }
    }
  }

  fence_before_sync();
  __syncthreads();
  __syncwarp();
  if (CG == 2) cluster_sync_all();
  if (warp == 1) {
    fence_after_sync();
    if (CG == 2) tmem_dealloc_pair(tmem_base, 512); else tmem_dealloc(tmem_base, 512);
  }
}

template <int CG>
static int launch(const CUtensorMap& mg, const CUtensorMap& mx, const WgradParams& p, int ctas, cudaStream_t st) {
  if (cudaFuncSetAttribute(grouped_wgrad_kernel<CG>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
    return 4;
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CG;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int units = ctas / CG;
  if (CG == 2) {
    static int resident = -1;
    if (resident < 0) {
      cfg.gridDim = dim3(2, 1, 1);
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, grouped_wgrad_kernel<CG>, &cfg) != cudaSuccess) n = 0;
      resident = n;
    }
    if (resident < 1) return 5;
    if (units > resident) units = resident;
  }
  if (units < 1) units = 1;
  cfg.gridDim = dim3(units * CG, 1, 1);
  return cudaLaunchKernelEx(&cfg, grouped_wgrad_kernel<CG>, mg, mx, p) == cudaSuccess ? 0 : 5;
}

}  // namespace wg

int launch_grouped_wgrad(const void* g, const void* x, long long rows, WgradParams p, int ctas, bool pair,
                         cudaStream_t st) {
  const int tm = pair ? 256 : 128;
  // pairs split a 256-row tile of dW between two CTAs: M % 256; a single CTA masks a ragged last tile: M % 8
  if (p.El < 1 || p.El > wg::kMaxLocalExperts || p.M <= 0 || (pair ? p.M % tm : p.M % 8) || p.N <= 0 || p.N % 8) return 1;
  if (reinterpret_cast<uintptr_t>(g) % 16 || reinterpret_cast<uintptr_t>(x) % 16 || rows < 1) return 1;
  CUtensorMap mg, mx;
  if (make_tmap_bf16(&mg, g, rows, p.M, 64, wg::BK)) return 3;
  if (make_tmap_bf16(&mx, x, rows, p.N, 64, wg::BK)) return 3;
  p.max_rows = (int)rows;
  if (ctas < 1) ctas = 1;
  return pair ? wg::launch<2>(mg, mx, p, ctas, st) : wg::launch<1>(mg, mx, p, ctas, st);
}

}  // namespace b200ep
