// Host-callable launchers of the copy kernels. Every launcher validates its arguments
// (alignment, sizes, limits) and returns 0 on success, non-zero when it refused to launch.
#pragma once
#include <cuda_runtime.h>

namespace b200ep {

// dst[0:n] = src[0:n], `iters` times inside one launch (persistent mode when iters > 1).
// vec_bytes: 16 or 32 (falls back to 16, then to bytes, when pointers are not aligned).
int launch_lsu_copy(void* dst, const void* src, long long nbytes, int ctas, int threads,
                    int iters, int vec_bytes, cudaStream_t st);

// Chunk c = offset / rr_bytes of the source goes to dsts[c % n_dst] at the same offset.
int launch_lsu_rr_copy(void* const* dsts, int n_dst, const void* src, long long nbytes,
                       long long rr_bytes, int ctas, int threads, int iters, cudaStream_t st);

// Shared-memory staged copy. pull = 0: src is LOCAL, dsts may be peers (rr_bytes = 0 for a
// single destination). pull = 1: src may be a peer, dsts[0] is LOCAL.
// tile = bytes per stage, piece = bytes per bulk store (pull), threads = 32 + consumer threads.
int launch_tma_staged_copy(void* const* dsts, int n_dst, const void* src, long long nbytes,
                           long long rr_bytes, int pull, int tile, int piece, int stages, int ctas,
                           int threads, int iters, int* status, cudaStream_t st);

// Broadcast src[0:n] to offset 0.. of EVERY GPU bound to the multicast address mc_dst
// (16-byte multiples, `multimem.st`). The caller orders completion (stream sync + barrier).
int launch_multimem_bcast(void* mc_dst, const void* src, long long nbytes, int ctas, int threads, int iters,
                          cudaStream_t st);

// One launch that performs a table of independent copies (the SM stand-in for a batched
// memcpy submission). desc is a DEVICE array of n entries.
struct CopyDesc { void* dst; const void* src; long long nbytes; };
int launch_batched_copy(const CopyDesc* desc_dev, int n, int ctas_per_copy, int threads,
                        cudaStream_t st);

}  // namespace b200ep
