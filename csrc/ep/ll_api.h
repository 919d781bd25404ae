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
  long long count[2];         // unsigned [El] per parity: rows taken so far in each local expert's block
  long long recv_x[2];        // [0]: [El][R*M][row_bytes] rows packed per local expert, in arrival order
  long long recv_scales[2];   // [0]: float [El][R*M][H/128]
  long long recv_src[2];      // [0]: int [El][R*M]  (source rank << 24 | token << 5 | k)
  long long comb_x[2];        // bf16 [M][K][H] per parity (push-form combine slots)
  long long recv_tag[2];      // unused
  long long comb_in;          // bf16 [El][R*M][H]  expert output written in place (pull-form combine), one copy
  long long range_tab[2];     // unused
  int G;                      // CTAs of EVERY dispatch-send launch (same on all ranks)
  int Gc;                     // CTAs of EVERY combine-send launch (multiple of El)
  int signal_mode;            // 0: every send CTA signals every peer; 1: the last CTA does (see ll.cu)
  int pdl;                    // 1: launch with programmatic stream serialisation (launch latencies overlap)
  unsigned long long timeout_ns;
};

// `state`: device int[6] per op (see ll.cu). `send_cnt`: device int[2*E], zero-initialised once.
// send_slot (optional): int [M*K], receives the slot given to every item (t,k), -1 = not sent.
void launch_ll_dispatch_send(const LLParams& P, const PeerPtrs& peers, const char* x,
                             const long long* topk_idx, int* send_cnt, int* state, int* status,
                             cudaStream_t st, int* send_slot = nullptr);
// Waits for every source's arrival and writes the rows per local expert to out_count [El].
void launch_ll_dispatch_recv(const LLParams& P, char* self_base, int* out_count, int* state, int* status,
                             cudaStream_t st);
void launch_ll_combine_send(const LLParams& P, const PeerPtrs& peers, const char* x, const int* src_info,
                            const int* count, int* state, int* status, cudaStream_t st);
// Pull form of the low-latency combine: the expert output stays in the producers' regions
// (`comb_in`, row (e, j) matching row (e, j) of the dispatched rows); every rank announces that its
// output is complete, waits for the peers, then loads the K rows of each of its tokens over NVLink
// and reduces them with the routing weights. phase 0: one launch; 1: announce only; 2: wait +
// reduce (two launches only for several virtual ranks on one GPU). send_slot: int [M*K], the
// packed row that dispatch took for item (t,k) on its destination, -1 = dropped. state: device int[6].
void launch_ll_combine_pull(const LLParams& P, const PeerPtrs& peers, int phase, const int* send_slot,
                            const long long* topk_idx, const float* topk_w, char* out, int* state,
                            int* status, cudaStream_t st);

void launch_ll_combine_recv(const LLParams& P, char* self_base, const long long* topk_idx,
                            const float* topk_w, char* out, int* state, int* status,
                            int blocks, cudaStream_t st);

}  // namespace b200ep
