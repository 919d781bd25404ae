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
// GPU's memory, no cluster multicast), warp 1 = MMA issuer and TMEM owner, warps 2-5 = epilogue.
// 4-stage smem ring (A 128x64 + B 256x64 bf16, 128-byte swizzle), 2 TMEM accumulators
// (128 lanes x 256 f32 columns each) so the epilogue of tile i overlaps the MMAs of tile i+1.
// The tile list is derived on the device from the per-expert row offsets (no host sync).
// Every mbarrier wait is bounded; on a time-out all roles leave their loops, TMEM is freed.
#include <cuda_bf16.h>
#include "tc05.cuh"
#include "gemm_api.h"

namespace b200ep {

using namespace tc;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_HALF_BYTES = 128 * BK * 2, STAGE_BYTES = A_BYTES + 2 * B_HALF_BYTES;
constexpr int EPI_ROW_BYTES = 128 + 16;                       // 64 bf16 + pad (bank spread)
constexpr int EPI_WARP_BYTES = 32 * EPI_ROW_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 4 * EPI_WARP_BYTES + 1024 /*align slack*/;
constexpr int GEMM_THREADS = 192;
constexpr int kMaxLocalExperts = 256;

struct Tile { int e, row0, valid_rows, nt; };

// Tile t -> (expert, first row, valid rows, n-tile). Tiles of one expert are consecutive,
// m fastest, so CTAs that run together share the same weight tile in L2.
__device__ __forceinline__ bool decode_tile(int t, const int* s_tile_off, const int* s_row_off, int El,
                                            int n_tiles, Tile& out) {
  if (t >= s_tile_off[El]) return false;
  int e = 0;
  while (e + 1 < El && t >= s_tile_off[e + 1]) ++e;
  const int local = t - s_tile_off[e];
  const int rows = s_row_off[e + 1] - s_row_off[e];
  const int m_tiles = (rows + BM - 1) / BM;
  const int mt = local % m_tiles;
  out.e = e;
  out.nt = local / m_tiles;
  out.row0 = s_row_off[e] + mt * BM;
  out.valid_rows = min(BM, rows - mt * BM);
  (void)n_tiles;
  return true;
}

__device__ __forceinline__ float silu(float v) { return v / (1.f + __expf(-v)); }

template <int EPI>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ GemmParams p, const __grid_constant__ PeerPtrs peers) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ int s_tile_off[kMaxLocalExperts + 1], s_row_off[kMaxLocalExperts + 1];

  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* epi_smem = smem + STAGES * STAGE_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort = &s_abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
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
      acc += ((r1 - r0 + BM - 1) / BM) * p.n_tiles;
    }
    s_tile_off[p.El] = acc;
    prefetch_tmap(&map_a);
    prefetch_tmap(&map_b);
  }
  if (warp == 1) tmem_alloc(&s_tmem, 512);
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = s_tmem;
  const int k_blocks = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      uint32_t it = 0;
      Tile tl;
      for (int t = blockIdx.x; decode_tile(t, s_tile_off, s_row_off, p.El, p.n_tiles, tl) && !*abort; t += gridDim.x) {
        const int b_row0 = (EPI == EPI_SWIGLU) ? tl.e * p.w_rows + tl.nt * 128 : tl.e * p.w_rows + tl.nt * BN;
        const int b_row1 = (EPI == EPI_SWIGLU) ? b_row0 + p.N : b_row0 + 128;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (it >= STAGES && !mbar_wait(&empty_bar[s], ph ^ 1, p.status, abort)) break;
          unsigned char* st = smem + s * STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          tma_load_2d(st, &map_a, kb * BK, tl.row0, &full_bar[s]);
          tma_load_2d(st + A_BYTES, &map_b, kb * BK, b_row0, &full_bar[s]);
          tma_load_2d(st + A_BYTES + B_HALF_BYTES, &map_b, kb * BK, b_row1, &full_bar[s]);
        }
      }
      if (*abort) {
        // let my own loads that are still in flight land before the CTA's shared memory goes away
        int quiet = 0;
        for (uint32_t n = it > STAGES ? it - STAGES : 0; n < it; ++n)
          mbar_wait(&full_bar[n % STAGES], (n / STAGES) & 1, nullptr, &quiet);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      const uint32_t idesc = instr_desc_bf16(BM, BN);
      uint32_t it = 0, tile_n = 0;
      Tile tl;
      for (int t = blockIdx.x; decode_tile(t, s_tile_off, s_row_off, p.El, p.n_tiles, tl) && !*abort; t += gridDim.x, ++tile_n) {
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
          const uint64_t a_desc = smem_desc_sw128(a_addr), b_desc = smem_desc_sw128(a_addr + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)   // 16 bf16 = 32 bytes per MMA step: +2 in 16-byte units
            mma_bf16(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) ? 1u : 0u);
          mma_commit(&empty_bar[s]);          // frees the smem stage when these MMAs retire
        }
        if (!ok) break;
        mma_commit(&acc_full[buf]);           // accumulator complete
      }
    }
  } else {
    // ---------------- epilogue (4 warps, one TMEM lane quarter each) ----------------
    const int q = warp & 3;                        // TMEM lanes [32q, 32q+32)
    unsigned char* my_smem = epi_smem + (warp - 2) * EPI_WARP_BYTES;
    uint32_t tile_n = 0;
    Tile tl;
    for (int t = blockIdx.x; decode_tile(t, s_tile_off, s_row_off, p.El, p.n_tiles, tl) && !*abort; t += gridDim.x, ++tile_n) {
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
      for (int c = 0; c < OUT_COLS / 64; ++c) {
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
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }

  // ---------------- teardown: every path arrives here ----------------
  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, 512);
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
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 2-D bf16 tensor [rows, cols] (cols contiguous), box = 64 cols x 128 rows, 128-byte swizzle.
static int make_map(CUtensorMap* m, const void* base, long long rows, long long cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return 1;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {BK, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2;
}

int launch_grouped_gemm(const void* a, long long a_rows, const void* w, int epi, GemmParams p,
                        const PeerPtrs& peers, int ctas, cudaStream_t st) {
  if (p.El < 1 || p.El > kMaxLocalExperts || p.K <= 0 || p.K % 8 || p.N <= 0 || p.N_out % 8) return 1;
  if (reinterpret_cast<uintptr_t>(a) % 16 || reinterpret_cast<uintptr_t>(w) % 16) return 1;
  if (epi == EPI_SWIGLU && (p.N % 128)) return 1;
  CUtensorMap ma, mb;
  if (make_map(&ma, a, a_rows, p.K)) return 3;
  if (make_map(&mb, w, (long long)p.El * p.w_rows, p.K)) return 3;
  p.n_tiles = epi == EPI_SWIGLU ? p.N / 128 : (p.N + BN - 1) / BN;
  p.max_rows = (int)a_rows;
  if (ctas < 1) ctas = 1;
  cudaError_t e;
#define B200EP_GEMM_LAUNCH(EPI)                                                                          \
  e = cudaFuncSetAttribute(grouped_gemm_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES); \
  if (e != cudaSuccess) return 4;                                                                        \
  grouped_gemm_kernel<EPI><<<ctas, GEMM_THREADS, SMEM_BYTES, st>>>(ma, mb, p, peers)
  if (epi == EPI_PLAIN) { B200EP_GEMM_LAUNCH(EPI_PLAIN); }
  else if (epi == EPI_SWIGLU) { B200EP_GEMM_LAUNCH(EPI_SWIGLU); }
  else if (epi == EPI_COMBINE) { B200EP_GEMM_LAUNCH(EPI_COMBINE); }
  else return 1;
  return 0;
}

}  // namespace b200ep
