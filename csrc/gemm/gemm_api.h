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
  int w_rows;             // rows per expert in the weight tensor (N, or 2F for swiglu)
  int n_tiles, max_rows;  // filled by the launcher
  const int* expert_off;  // device [El+1]: exclusive prefix of rows per local expert
  void* out;              // bf16 [rows, out_ld]           (plain / swiglu)
  long long out_ld;
  const float* row_prob;  // f32 [rows] or null            (swiglu)
  const int2* recv_meta;  // {slot at source, source rank} (combine)
  long long comb_off;     // offset of the combine region in every rank's symmetric buffer
  int slot_cap, R, rank;
  long long signal_flag_off;   // offset of the combine flag row (< 0: do not signal)
  unsigned int* block_counter;
  int epoch;
  int* status;
};

// a: bf16 [a_rows, K] on this GPU; w: bf16 [El * w_rows, K] on this GPU. Returns 0 on success.
int launch_grouped_gemm(const void* a, long long a_rows, const void* w, int epi, GemmParams p,
                        const PeerPtrs& peers, int ctas, cudaStream_t st);

}  // namespace b200ep
