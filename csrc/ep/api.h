// Host-callable launchers of the EP kernels (raw pointers + stream; no torch types, so the
// .cu files compile in seconds and can also be linked from plain C++).
#pragma once
#include <cuda_runtime.h>
#include "ep.cuh"

namespace b200ep {

void launch_layout(const long long* topk_idx, int T, int K, int E, int R, int* per_rank,
                   int* per_expert, bool* in_rank, int* status, cudaStream_t st);

void launch_notify_send(const EpGeom& g, const EpRegions& rg, const PeerPtrs& peers,
                        const bool* is_in_rank, const long long* topk_idx,
                        const int* num_tokens_per_expert, int* item_rank, int* chunk_hist,
                        unsigned int* block_counter, int* status, cudaStream_t st);

void launch_notify_wait(const EpGeom& g, const EpRegions& rg, char* self_base, const EpMeta& m,
                        int* host_word, int* status, cudaStream_t st);

void launch_wait_flags(char* self_base, long long flags_off, int channel, int R, int epoch,
                       unsigned long long timeout_ns, int* status, int code, cudaStream_t st);

void launch_barrier(const PeerPtrs& peers, long long flags_off, int rank, int R, int epoch,
                    unsigned long long timeout_ns, int* status, int wait, cudaStream_t st);

void launch_dispatch_send(const EpGeom& g, const EpRegions& rg, const PeerPtrs& peers,
                          const EpMeta& m, const char* x, int row_bytes_in, bool fp8, bool cached,
                          const long long* topk_idx, const float* topk_w, const int* item_rank,
                          const int* chunk_base, int* send_row, int* send_slot,
                          unsigned int* block_counter, int* status, int blocks, cudaStream_t st,
                          const float* scales_in = nullptr);

void launch_combine_send(const EpGeom& g, const EpRegions& rg, const PeerPtrs& peers,
                         const int* n_recv_ptr, const int* recv_meta, const char* x, int row_bytes,
                         const float* topk_w, unsigned int* block_counter, int* status, int blocks,
                         cudaStream_t st);

void launch_signal(const PeerPtrs& peers, long long flags_off, int channel, int rank, int R,
                   int epoch, cudaStream_t st);

void launch_combine_reduce(const EpGeom& g, const EpRegions& rg, char* self_base,
                           const int* send_slot, const float* weights, char* out, float* out_topk_w,
                           int dtype_code, int wait_epoch, int* status, int blocks, cudaStream_t st);

}  // namespace b200ep
