// Host-callable launchers of the EP kernels (raw pointers + stream; no torch types, so the
// .cu files compile in seconds and can also be linked from plain C++).
#pragma once
#include <cuda_runtime.h>
#include "ep.cuh"

namespace b200ep {

// Ints of scratch that launch_layout needs (`partial`), for T tokens.
int layout_scratch_ints(int T, int E, int R);

// `partial`: scratch of layout_scratch_ints(...) ints; `block_counter`: one zero-initialised word
// that the kernel leaves at zero. Outputs need no zero-fill.
void launch_layout(const long long* topk_idx, int T, int K, int E, int R, int* per_rank,
                   int* per_expert, bool* in_rank, int* partial, unsigned int* block_counter,
                   int* status, cudaStream_t st);

void launch_notify_send(const EpGeom& g, const EpRegions& rg, const PeerPtrs& peers,
                        const bool* is_in_rank, const long long* topk_idx,
                        const int* num_tokens_per_expert, int* item_rank, int* chunk_hist,
                        unsigned int* block_counter, int* status, cudaStream_t st);

void launch_wait_flags(char* self_base, long long flags_off, int channel, int R, int epoch,
                       unsigned long long timeout_ns, int* status, int code, cudaStream_t st);

void launch_barrier(const PeerPtrs& peers, long long flags_off, int rank, int R, int epoch,
                    unsigned long long timeout_ns, int* status, int wait, cudaStream_t st);

// g.epoch = dispatch epoch to publish, g.epoch_wait = notify epoch to wait for (fresh dispatch),
// g.tail_wait = 1 makes the last CTA wait for the peers' dispatch flags (never with several
// virtual ranks on one GPU: use launch_wait_flags on the dispatch channel after all ranks' sends).
// host_word: mapped pinned ints [0]=notify epoch served, [1]=N_recv, [2..2+El) per-expert counts.
void launch_dispatch_send(const EpGeom& g, const EpRegions& rg, const PeerPtrs& peers,
                          const EpMeta& m, const char* x, int row_bytes_in, bool fp8, bool cached,
                          const long long* topk_idx, const float* topk_w, const int* item_rank,
                          const int* chunk_base, int* send_row, int* send_slot,
                          unsigned int* block_counter, int* host_word, int* status, int blocks,
                          cudaStream_t st, const float* scales_in = nullptr);

enum CombineRole : int { kCombineBoth = 0, kCombineSendOnly = 1, kCombineReduceOnly = 2 };

// Push form of combine (see combine.cu). kCombineBoth: every CTA sends its share of the rows, then
// waits for the peers' flags and reduces its share of the tokens (one process per GPU only).
struct CombineArgs {
  int role;                  // CombineRole
  // send role
  const int* n_recv_ptr;     // device: number of valid rows in x
  const int2* recv_meta;     // [n_recv] {slot at source, source rank}
  const char* x;             // [n_recv][row_bytes]
  int row_bytes;
  const float* topk_w;       // optional side values returned with the rows
  unsigned int* block_counter;  // zero on entry, left at zero
  // reduce role
  int wait;                  // 1: wait for every rank's combine flag of g.epoch first
  const int* send_slot;      // [T][J]
  const float* weights;      // optional [T][J]
  char* out;                 // [T][H]
  float* out_topk_w;         // optional [T][K]
};

// Number of SMs: the largest useful grid (CTAs have 1024 threads, one per SM).
int combine_max_ctas();

// dtype_code: 0 bf16, 1 fp16, 2 fp32 (element type of x / out).
void launch_combine(const EpGeom& g, const EpRegions& rg, const PeerPtrs& peers, const CombineArgs& a,
                    int dtype_code, int* status, int blocks, cudaStream_t st);

// Pull form of combine: the rows to be combined stay where their producer wrote them, inside the
// producer's symmetric region; every rank tells its peers where (`publish`), waits for the peers'
// announcements and then LOADS the rows of its own tokens over NVLink, reducing them in registers.
// No slot region, no second pass over the rows, nothing left to do when the last row has arrived.
struct CombinePullArgs {
  long long x_off;           // byte offset of MY rows inside my region (published to the peers)
  long long w_off;           // byte offset of my side values (float), or -1
  long long n_rows;          // rows that peers may read from x_off
  int publish;               // 1: announce x_off / w_off / n_rows and raise my flag on every peer
  int wait;                  // 1: wait for every peer's announcement of this epoch
  int pull;                  // 1: do the reduction (0 = announce only)
  const int* send_row;       // [T][J] row of (token, item) at its destination
  const long long* topk_idx; // [T][K] (expert mode: which rank holds item k)
  const float* weights;      // optional [T][J]
  char* out;                 // [T][H]
  float* out_topk_w;         // optional [T][K]
};
void launch_combine_pull(const EpGeom& g, const EpRegions& rg, const PeerPtrs& peers,
                         const CombinePullArgs& a, int dtype_code, int* status, int blocks, cudaStream_t st);

void launch_signal(const PeerPtrs& peers, long long flags_off, int channel, int rank, int R,
                   int epoch, cudaStream_t st);

}  // namespace b200ep
