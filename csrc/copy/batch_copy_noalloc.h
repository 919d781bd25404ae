// b200ep_batched_copy_noalloc: a batched device copy for callers that must not allocate.
//
// This entry point has no counterpart in the reference benchmark suite; it exists for users of
// this library only.
//
// Who needs it: code that runs where device allocation is forbidden or impossible, e.g. a
// plug-in called from inside another framework's memory plan (every byte of device memory is
// already handed out and an allocation would fail or fragment the plan), a latency-critical
// serving loop in which an allocation could synchronise the device, or a host thread that is
// not allowed to touch the allocator. The regular path (`CeEngine` in kernel mode,
// `launch_batched_copy`) keeps its table of copy descriptors in memory obtained with cudaMalloc;
// this variant keeps the table in a fixed array that is part of the library image instead.
//
// Contract
//  * Performs n independent copies dsts[i][0:sizes[i]) = srcs[i][0:sizes[i]) with one kernel
//    launch on `stream`. Inputs and outputs are the caller's; the only extra memory is the
//    descriptor table described below.
//  * Limit: n <= B200EP_NOALLOC_MAX_COPIES (1024). Larger n, n <= 0, a null array, a negative
//    size or a bad launch shape is rejected with a negative return code and nothing is launched;
//    `b200ep_noalloc_error_string` turns the code into text.
//  * Scratch: one file-scope device array of 1024 descriptors (24 KiB, 256-byte aligned). Every
//    GPU that loads the library carries its own copy until the process exits.
//  * The first call on a given device looks up the array's device address (with that device
//    current) and remembers it; make that first call before starting any stream capture.
//  * The call itself must not be made on a stream that is being captured: the descriptors are
//    uploaded from this function's stack, which a captured copy node would keep pointing at.
//    Such a call is refused with code -7 and nothing is issued.
//  * The upload is a copy from pageable memory: the calling host thread waits until earlier
//    work on `stream` has drained before the function returns.
//  * Every call overwrites the same table, which otherwise keeps the previous call's contents.
//    Calls issued to ONE stream are ordered and safe. Calls that may overlap on the GPU
//    (different streams, different host threads) race on the table: serialise them yourself.
//  * Neither this function nor anything it calls uses cudaMalloc, cudaFree or an allocating
//    library routine.
#pragma once
#include <cuda_runtime.h>

#define B200EP_NOALLOC_MAX_COPIES 1024

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0 on success; < 0: argument error (see b200ep_noalloc_error_string); > 0: a cudaError_t.
int b200ep_batched_copy_noalloc(void* const* dsts, const void* const* srcs, const long long* sizes, int n,
                                int ctas_per_copy, int threads, cudaStream_t stream);

const char* b200ep_noalloc_error_string(int code);

#ifdef __cplusplus
}
#endif
