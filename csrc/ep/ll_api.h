// Launchers of the low-latency kernels.
#pragma once
#include <cuda_runtime.h>
#include "ep.cuh"

namespace b200ep {

struct LLParams {
  int rank, R, E, El, K, H;
  int M;     // capacity: max tokens a rank dispatches per call
  int T;     // tokens of this call (<= M)
  int fp8;   // 1: e4m3 payload + 1x128 f32 scales, 0: bf16 payload
  long long flags;            // int [kNumChannels][kMaxRanks]
  long long count[2];         // int [El][R]               per parity
  long long recv_x[2];        // [El][R][M][row_bytes]
  long long recv_scales[2];   // float [El][R][M][H/128]
  long long recv_src[2];      // int [El][R][M]  (token << 5 | k)
  long long comb_x[2];        // bf16 [M][K][H]
  long long recv_tag[2];      // int [El][R][M]  epoch in which the slot was written
  int G;                      // CTAs of EVERY dispatch-send launch (same on all ranks)
  int Gc;                     // CTAs of EVERY combine-send launch (multiple of El)
  int signal_mode;            // 0: every send CTA signals every peer; 1: the last CTA does (see ll.cu)
  int pdl;                    // 1: launch with programmatic stream serialisation (launch latencies overlap)
  unsigned long long timeout_ns;
};

// `state`: device int[6] per op (see ll.cu). `send_cnt`: device int[2*E], zero-initialised once.
void launch_ll_dispatch_send(const LLParams& P, const PeerPtrs& peers, const char* x,
                             const long long* topk_idx, int* send_cnt, int* state, int* status,
                             cudaStream_t st);
void launch_ll_dispatch_recv(const LLParams& P, char* self_base, char* out_x, float* out_scales,
                             int* out_src, int* out_count, int* out_range, int* state,
                             int* status, int split, cudaStream_t st);
void launch_ll_combine_send(const LLParams& P, const PeerPtrs& peers, const char* x, const int* src_info,
                            const int* count, int* state, int* status, cudaStream_t st);
void launch_ll_combine_recv(const LLParams& P, char* self_base, const long long* topk_idx,
                            const float* topk_w, char* out, int* state, int* status,
                            int blocks, cudaStream_t st);

}  // namespace b200ep
