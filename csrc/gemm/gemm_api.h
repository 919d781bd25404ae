// Host launcher of the tcgen05 grouped GEMM.
#pragma once
#include <cuda_runtime.h>
#include "../common.cuh"

namespace b200ep {

enum GemmEpilogue : int { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_COMBINE = 2 };

struct GemmParams {
  int El;                 // local experts
  int N;                  // plain/combine: output features; swiglu: F (gate and linear blocks of F rows each)
  int K;                  // reduction length
  int N_out;              // columns of the stored result (== N)
  int w_rows;             // rows per expert in the weight tensor (N, or 2F for swiglu; K if b_mn)
  int b_mn;               // 1: weights stored [El, K, N] (N contiguous), plain epilogue only
  int n_tiles, max_rows;  // filled by the launcher
  int band_rows;          // activation rows per L2-resident band of the tile order (<= 0: 2048)
  const int* expert_off;  // device [El+1]: exclusive prefix of rows per local expert
  void* out;              // bf16 [rows, out_ld]           (plain / swiglu)
  long long out_ld;
  const float* row_prob;  // f32 [rows] or null            (swiglu)
  void* pre_out;          // bf16 [rows, pre_ld] or null   (swiglu: also store the pre-activation [gate | linear])
  long long pre_ld;
  const int2* recv_meta;  // {slot at source, source rank} (combine)
  long long comb_off;     // offset of the combine region in every rank's symmetric buffer
  int slot_cap, R, rank;
  long long signal_flag_off;   // offset of the combine flag row (< 0: do not signal)
  unsigned int* block_counter;
  int epoch;
  int* status;
};

// a: bf16 [a_rows, K] on this GPU; w: bf16 [El * w_rows, K] on this GPU. Returns 0 on success.
// pair: run CTA pairs (clusters of two SMs, `cta_group::2`) on 256 x 256 tiles instead of single
// CTAs on 128 x 256 tiles; `ctas` then counts CTAs as well (pairs = ctas / 2, capped by residency).
int launch_grouped_gemm(const void* a, long long a_rows, const void* w, int epi, GemmParams p,
                        const PeerPtrs& peers, int ctas, bool pair, cudaStream_t st);

// Block-scaled fp8 grouped GEMM (csrc/gemm/grouped_gemm_fp8.cu).
struct GemmFp8Params {
  int El;                 // local experts
  int N;                  // plain: output features; swiglu: F (gate and linear blocks of F weight rows each)
  int K;                  // reduction length (multiple of 128)
  int N_out;              // columns of the stored result (== N)
  int w_rows;             // weight rows per expert (N, or 2F for swiglu); multiple of 128
  int n_tiles, max_rows;  // filled by the launcher
  int band_rows;          // activation rows per L2-resident band of the tile order (<= 0: 2048)
  const int* expert_off;  // device [El+1]
  const float* sa;        // f32 [rows, sa_ld]: scale of row r, reduction block kb at sa[r * sa_ld + kb]
  long long sa_ld;
  const float* sw;        // f32 [El, w_rows / 128, K / 128]
  void* out;              // bf16 [rows, out_ld]
  long long out_ld;
  const float* row_prob;  // f32 [rows] or null (swiglu)
  int* status;
};
// a: e4m3 [a_rows, K], w: e4m3 [El * w_rows, K], both on this GPU. epi: EPI_PLAIN or EPI_SWIGLU.
int launch_grouped_gemm_fp8(const void* a, long long a_rows, const void* w, int epi, GemmFp8Params p, int ctas,
                            cudaStream_t st);

// Weight gradient of a grouped GEMM: dW[e] = G_e^T . X_e over the rows of local expert e.
struct WgradParams {
  int El;                 // local experts
  int M, N;               // dW[e] is [M, N]: M = columns of G, N = columns of X
  int max_rows;           // filled by the launcher
  const int* expert_off;  // device [El+1]
  void* out;              // bf16 [El, M, N]
  int* status;
};
// g: bf16 [rows, M], x: bf16 [rows, N], both on this GPU, rows grouped by local expert.
// pair: CTA pairs on 256 x 256 tiles of dW (M % 256 == 0) instead of single CTAs on 128 x 256 (M % 8 == 0; a
// last tile that hangs over M reads zeros and stores only the rows below M).
int launch_grouped_wgrad(const void* g, const void* x, long long rows, WgradParams p, int ctas, bool pair,
                         cudaStream_t st);

// SwiGLU x prob elementwise pair for the training path (h: bf16 [rows, 2F], gate columns first).
// n_rows_ptr (device, optional) bounds the rows actually processed; max_rows is the tensor's size.
int launch_swiglu_fwd(const void* h, const float* p, void* act, const int* n_rows_ptr, int max_rows, int F,
                      cudaStream_t st);
int launch_swiglu_bwd(const void* h, const float* p, const void* dact, void* dh, float* dp, const int* n_rows_ptr,
                      int max_rows, int F, cudaStream_t st);

// Ungated activation x prob pair (h: bf16 [rows, F]); kind: 0 gelu (erf form), 1 silu, 2 relu.
int launch_act_fwd(const void* h, const float* p, void* act, const int* n_rows_ptr, int max_rows, int F, int kind,
                   cudaStream_t st);
int launch_act_bwd(const void* h, const float* p, const void* dact, void* dh, float* dp, const int* n_rows_ptr,
                   int max_rows, int F, int kind, cudaStream_t st);

}  // namespace b200ep
