// Block-scaled fp8 (e4m3) grouped expert GEMM on the 5th-generation tensor cores.
//
//   out[r, :] = epilogue( sum_kb  sa[r, kb] * sw[e(r), nb, kb] * ( Aq[r, kb-block] . Wq[e(r)][:, kb-block]^T ) )
//
// Aq: e4m3 [rows, K] with one f32 scale per row and 128 channels (`sa`, [rows, K/128]): exactly what
// the fp8 dispatch writes into the receive region, so the expert consumes the dispatched rows
// without a dequantisation pass. Wq: e4m3 [E_local, N_w, K] with one f32 scale per 128 x 128 block
// (`sw`, [E_local, N_w/128, K/128]). Replaces the bf16 cast + library GEMM that the reference's
// expert MLP would need for fp8 inputs (`DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:528-541`).
//
// The tensor core multiplies raw e4m3 values (`tcgen05.mma kind::f8f6f4`, f32 accumulate); the
// scales differ per 128-wide reduction block, so every block's partial product is a SEPARATE
// accumulator in TMEM (two of 128 lanes x 256 columns, used alternately) which the epilogue warps
// read back, scale and add to an f32 running sum in registers ("promotion") while the tensor core
// already works on the next block. Structure per CTA (persistent, one per SM, 320 threads):
//   warp 0      TMA producer: per reduction block one 128 x 128-byte tile of A and one
//               256 x 128-byte tile of W (128-byte swizzle), 4-stage ring; plain loads of this
//               GPU's memory, every CTA fetches its own tiles.
//   warp 1      MMA issuer and TMEM owner: 4 MMAs (K = 32 each) per block, then two commits:
//               one frees the shared-memory stage, one announces the partial accumulator.
//   warps 2-9   promotion + epilogue: warp w works on TMEM lanes 32 * (w % 4) and on one half of
//               the columns (128 running sums per thread).
// Epilogues: plain bf16 store; SwiGLU x prob (weights hold [gate rows | linear rows], a tile
// multiplies 128 gate and the matching 128 linear rows; each thread keeps gate and linear sums of
// the same 64 output columns, so no exchange between threads is needed).
// Every mbarrier wait is bounded; on a time-out all roles leave their loops and TMEM is freed.
#include <cuda_bf16.h>
#include "tc05.cuh"
#include "tmap.h"
#include "gemm_api.h"

namespace b200ep {

using namespace tc;

namespace f8 {

constexpr int BM = 128, BN = 256, BKB = 128;                   // BKB: reduction block = 128 fp8 = 128 bytes
constexpr int A_BYTES = BM * BKB, B_BYTES = BN * BKB;          // 16 KiB + 32 KiB
constexpr int STAGES = 4, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int RING_BYTES = STAGES * STAGE_BYTES;               // 192 KiB
constexpr int EPI_WARPS = 8;
constexpr int EPI_COLS = 32;                                   // output columns per store pass
constexpr int EPI_ROW_BYTES = EPI_COLS * 2 + 16;               // 32 bf16 + pad (bank spread)
constexpr int EPI_WARP_BYTES = 32 * EPI_ROW_BYTES;
constexpr int SMEM_BYTES = RING_BYTES + EPI_WARPS * EPI_WARP_BYTES + 1024;
constexpr int THREADS = 64 + EPI_WARPS * 32;
constexpr int kMaxLocalExperts = 256;

struct Tile { int e, row0, valid_rows, nt; };

// Same tile order as the bf16 kernel: inside an expert, bands of `gm` m-tiles; inside a band m
// runs fastest, then n (the band of activation rows stays in L2 while the weight tiles pass).
__device__ __forceinline__ bool decode_tile(int t, const int* s_tile_off, const int* s_row_off, int El,
                                            int n_tiles, int gm, Tile& out) {
  if (t >= s_tile_off[El]) return false;
  int e = 0;
  while (e + 1 < El && t >= s_tile_off[e + 1]) ++e;
  const int local = t - s_tile_off[e];
  const int rows = s_row_off[e + 1] - s_row_off[e];
  const int m_tiles = (rows + BM - 1) / BM;
  const int per_band = gm * n_tiles;
  const int band = local / per_band;
  const int idx = local - band * per_band;
  const int band_m = min(gm, m_tiles - band * gm);
  const int mt = band * gm + idx % band_m;
  out.e = e;
  out.nt = idx / band_m;
  out.row0 = s_row_off[e] + mt * BM;
  out.valid_rows = max(0, min(BM, rows - mt * BM));
  return true;
}

__device__ __forceinline__ float silu(float v) { return __fdividef(v, 1.f + __expf(-v)); }

// e4m3 x e4m3 -> f32, K-major operands, tile M x N
__device__ __forceinline__ uint32_t instr_desc_e4m3(int M, int N) {
  return (1u << 4) /* f32 accumulator */ | (0u << 7) /* A: e4m3 */ | (0u << 10) /* B: e4m3 */ |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void mma_e4m3(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}"
      ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

template <int EPI>
__global__ void __launch_bounds__(THREADS, 1)
grouped_gemm_fp8_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ GemmFp8Params p) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES], part_full[2], part_empty[2];
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  __shared__ int s_tile_off[kMaxLocalExperts + 1], s_row_off[kMaxLocalExperts + 1];

  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* epi_smem = smem + RING_BYTES;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort = &s_abort;
  const int gm = max(1, p.band_rows / BM);
  const int k_blocks = p.K / BKB;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&part_full[b], 1); mbar_init(&part_empty[b], EPI_WARPS); }
    s_abort = 0;
    fence_barrier_init();
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

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      uint32_t it = 0;
      Tile tl;
      for (int t = blockIdx.x; decode_tile(t, s_tile_off, s_row_off, p.El, p.n_tiles, gm, tl) && !*abort; t += gridDim.x) {
        // weight rows of this tile: [gate 128 | linear 128] for swiglu, 256 consecutive rows otherwise
        const int b_first = (EPI == EPI_SWIGLU) ? tl.e * p.w_rows + tl.nt * 128 : tl.e * p.w_rows + tl.nt * BN;
        const int b_second = (EPI == EPI_SWIGLU) ? b_first + p.N : b_first + 128;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (it >= STAGES && !mbar_wait(&empty_bar[s], ph ^ 1, p.status, abort)) break;
          unsigned char* st = smem + s * STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          tma_load_2d(st, &map_a, kb * BKB, tl.row0, &full_bar[s]);
          tma_load_2d(st + A_BYTES, &map_b, kb * BKB, b_first, &full_bar[s]);
          tma_load_2d(st + A_BYTES + B_BYTES / 2, &map_b, kb * BKB, b_second, &full_bar[s]);
        }
      }
      if (*abort) {
        // let the loads that are still in flight land before the CTA's shared memory goes away
        int quiet = 0;
        for (uint32_t n = it > STAGES ? it - STAGES : 0; n < it; ++n)
          mbar_wait(&full_bar[n % STAGES], (n / STAGES) & 1, nullptr, &quiet);
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: one partial accumulator per reduction block ----------------
    if (elect_one()) {
      const uint32_t idesc = instr_desc_e4m3(BM, BN);
      uint32_t it = 0;
      Tile tl;
      for (int t = blockIdx.x; decode_tile(t, s_tile_off, s_row_off, p.El, p.n_tiles, gm, tl) && !*abort; t += gridDim.x) {
        bool ok = true;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const int buf = it & 1;
          const uint32_t use = it >> 1;
          if (use > 0 && !mbar_wait(&part_empty[buf], (use - 1) & 1, p.status, abort)) { ok = false; break; }
          if (!mbar_wait(&full_bar[s], (it / STAGES) & 1, p.status, abort)) { ok = false; break; }
          fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t a_desc = smem_desc_sw128(a_addr);
          const uint64_t b_desc = smem_desc_sw128(a_addr + A_BYTES);
          const uint32_t d_tmem = tmem_base + buf * BN;
#pragma unroll
          for (int k = 0; k < BKB / 32; ++k)      // 32 e4m3 per MMA: +32 bytes = 2 descriptor units
            mma_e4m3(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, k ? 1u : 0u);
          mma_commit(&empty_bar[s]);              // the stage may be refilled when these MMAs retire
          mma_commit(&part_full[buf]);            // ... and the partial accumulator may be read
        }
        if (!ok) break;
      }
    }
  } else {
    // ---------------- promotion + epilogue: 8 warps = 4 lane quarters x 2 column halves ----------------
    const int ew = warp - 2;
    const int q = warp & 3;                        // TMEM lanes [32q, 32q+32) (a warp may only touch its own quarter)
    const int half = ew >> 2;                      // which half of the columns
    unsigned char* my_smem = epi_smem + ew * EPI_WARP_BYTES;
    uint32_t it = 0;
    Tile tl;
    const int kb_ld = p.sa_ld;
    for (int t = blockIdx.x; decode_tile(t, s_tile_off, s_row_off, p.El, p.n_tiles, gm, tl) && !*abort; t += gridDim.x) {
      const int my_row = tl.row0 + q * 32 + lane;
      const bool row_ok = q * 32 + lane < tl.valid_rows;
      // plain: my 128 columns are one 128-wide weight block; swiglu: 64 gate + the matching 64 linear columns
      const int col_a = (EPI == EPI_SWIGLU) ? half * 64 : half * 128;           // first TMEM column, group A
      const int col_b = (EPI == EPI_SWIGLU) ? 128 + half * 64 : half * 128 + 64;  // second group of 64 columns
      // (a last plain tile may hang over the expert's weight rows: its extra columns are never stored,
      // the scale index is clamped so that it stays inside the expert's scale rows)
      const int wblk_a = (EPI == EPI_SWIGLU) ? tl.nt : min(tl.nt * 2 + half, p.w_rows / 128 - 1);
      const int wblk_b = (EPI == EPI_SWIGLU) ? p.N / 128 + tl.nt : wblk_a;
      const float* sw_a = p.sw + ((size_t)tl.e * (p.w_rows / 128) + wblk_a) * k_blocks;
      const float* sw_b = p.sw + ((size_t)tl.e * (p.w_rows / 128) + wblk_b) * k_blocks;
      const float* sa_row = p.sa + (size_t)my_row * kb_ld;
      // the row's routing probability is needed only after the last block: fetch it now
      float prob = 1.f;
      if (EPI == EPI_SWIGLU && row_ok && p.row_prob) prob = __ldg(p.row_prob + my_row);
      float acc[128];
#pragma unroll
      for (int i = 0; i < 128; ++i) acc[i] = 0.f;
      float sa_next = row_ok ? __ldg(sa_row) : 0.f;
      bool ok = true;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const int buf = it & 1;
        const float sa_cur = sa_next;
        if (kb + 1 < k_blocks && row_ok) sa_next = __ldg(sa_row + kb + 1);
        const float fa = sa_cur * __ldg(sw_a + kb), fb = sa_cur * __ldg(sw_b + kb);
        if (!mbar_wait(&part_full[buf], (it >> 1) & 1, p.status, abort)) { ok = false; break; }
        fence_after_sync();
        const uint32_t t_addr = tmem_base + buf * BN + ((uint32_t)(q * 32) << 16);
        // four loads of 32 columns, software-pipelined: the next load is in flight while the
        // previous one is folded into the running sums
        const uint32_t c0 = t_addr + col_a, c1 = t_addr + col_a + 32, c2 = t_addr + col_b, c3 = t_addr + col_b + 32;
        uint32_t v0[32], v1[32];
        tmem_ld32(c0, v0);
        tmem_ld_wait();
        tmem_ld_pin(v0);
        tmem_ld32(c1, v1);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = fmaf(fa, __uint_as_float(v0[i]), acc[i]);
        tmem_ld_wait();
        tmem_ld_pin(v1);
        tmem_ld32(c2, v0);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[32 + i] = fmaf(fa, __uint_as_float(v1[i]), acc[32 + i]);
        tmem_ld_wait();
        tmem_ld_pin(v0);
        tmem_ld32(c3, v1);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[64 + i] = fmaf(fb, __uint_as_float(v0[i]), acc[64 + i]);
        tmem_ld_wait();
        tmem_ld_pin(v1);
        // every TMEM read of this block is done: hand the buffer back BEFORE the last fold
        fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&part_empty[buf]);
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[96 + i] = fmaf(fb, __uint_as_float(v1[i]), acc[96 + i]);
      }
      if (!ok) break;
      if (tl.valid_rows <= 0) continue;
      // ---- store: EPI_COLS output columns per pass through the per-warp staging tile ----
      constexpr int PASSES = ((EPI == EPI_SWIGLU) ? 64 : 128) / EPI_COLS;
#pragma unroll
      for (int ps = 0; ps < PASSES; ++ps) {
        uint32_t packed[EPI_COLS / 2];
#pragma unroll
        for (int i = 0; i < EPI_COLS / 2; ++i) {
          const int c = ps * EPI_COLS + 2 * i;
          float a0, a1;
          if (EPI == EPI_SWIGLU) {
            a0 = silu(acc[c]) * acc[64 + c] * prob;
            a1 = silu(acc[c + 1]) * acc[64 + c + 1] * prob;
          } else {
            a0 = acc[c];
            a1 = acc[c + 1];
          }
          __nv_bfloat162 hh = __floats2bfloat162_rn(a0, a1);
          packed[i] = *reinterpret_cast<uint32_t*>(&hh);
        }
        uint4* srow = reinterpret_cast<uint4*>(my_smem + lane * EPI_ROW_BYTES);
#pragma unroll
        for (int i = 0; i < EPI_COLS / 8; ++i)
          srow[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
        __syncwarp();
        const int col0 = ((EPI == EPI_SWIGLU) ? tl.nt * 128 + half * 64 : tl.nt * BN + half * 128) + ps * EPI_COLS;
        // coalesced: 4 lanes write one row's 64 bytes, 8 rows per step
#pragma unroll
        for (int step = 0; step < 4; ++step) {
          const int r = step * 8 + (lane >> 2);
          const int seg = lane & 3;
          if ((q * 32 + r) < tl.valid_rows && (col0 + seg * 8) < p.N_out) {
            const uint4 val = *reinterpret_cast<const uint4*>(my_smem + r * EPI_ROW_BYTES + seg * 16);
            char* dst = reinterpret_cast<char*>(p.out) + ((size_t)(tl.row0 + q * 32 + r) * p.out_ld + col0 + seg * 8) * 2;
            st_global_v4(dst, val);
          }
        }
        __syncwarp();
      }
    }
  }

  // ---------------- teardown: every path arrives here ----------------
  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// uint8 tensor [rows, cols] (cols contiguous); box = 128 bytes x box_rows, 128-byte swizzle
static int make_map_u8(CUtensorMap* m, const void* base, long long rows, long long cols, int box_rows) {
  EncodeTiledFn fn = tmap_encode_fn();
  if (!fn) return 1;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols};
  cuuint32_t box[2] = {(cuuint32_t)BKB, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2;
}

template <int EPI>
static int launch_one(const CUtensorMap& ma, const CUtensorMap& mb, const GemmFp8Params& p, int ctas, cudaStream_t st) {
  if (cudaFuncSetAttribute(grouped_gemm_fp8_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
    return 4;
  grouped_gemm_fp8_kernel<EPI><<<ctas, THREADS, SMEM_BYTES, st>>>(ma, mb, p);
  return 0;
}

}  // namespace f8

int launch_grouped_gemm_fp8(const void* a, long long a_rows, const void* w, int epi, GemmFp8Params p, int ctas,
                            cudaStream_t st) {
  using namespace f8;
  if (p.El < 1 || p.El > kMaxLocalExperts || p.K <= 0 || p.K % BKB || p.N <= 0 || p.N % 128 || p.N_out % 8) return 1;
  if (p.w_rows % 128 || p.sa == nullptr || p.sw == nullptr || p.sa_ld < p.K / BKB) return 1;
  if (reinterpret_cast<uintptr_t>(a) % 16 || reinterpret_cast<uintptr_t>(w) % 16) return 1;
  if (epi != EPI_PLAIN && epi != EPI_SWIGLU) return 1;
  CUtensorMap ma, mb;
  if (make_map_u8(&ma, a, a_rows, p.K, BM)) return 3;
  if (make_map_u8(&mb, w, (long long)p.El * p.w_rows, p.K, 128)) return 3;
  p.n_tiles = epi == EPI_SWIGLU ? p.N / 128 : (p.N + BN - 1) / BN;
  p.max_rows = (int)a_rows;
  if (p.band_rows <= 0) p.band_rows = 2048;
  if (ctas < 1) ctas = 1;
  if (epi == EPI_PLAIN) return launch_one<EPI_PLAIN>(ma, mb, p, ctas, st);
  return launch_one<EPI_SWIGLU>(ma, mb, p, ctas, st);
}

}  // namespace b200ep
