// One-to-all broadcast through the NVSwitch multicast address of a symmetric buffer: every
// 16-byte `multimem.st` is replicated by the switch into the same offset of EVERY GPU of the
// multicast group, so the source's NVLink carries the payload once instead of once per peer.
// This is the fan-out pattern of `Copy_Engine/nvlink_all_to_all_copy_engine_test.py:207-210`
// (one source buffer copied to a private buffer on every other GPU) done with one store stream.
// The multicast address comes from the caller (the NVLS-capable symmetric-memory allocator);
// nothing here reads through it, and no TMA is involved.
#include "../common.cuh"
#include "copy_api.h"

namespace b200ep {

__device__ __forceinline__ void multimem_st_v4(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(mc), "f"(__uint_as_float(v.x)), "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)),
                 "f"(__uint_as_float(v.w)) : "memory");
}

__global__ void multimem_bcast_kernel(char* mc_dst, const char* __restrict__ src, long long nbytes, int iters) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  const long long nvec = nbytes >> 4;
  for (int it = 0; it < iters; ++it) {
    long long v = tid;
    for (; v + 3 * nth < nvec; v += 4 * nth) {
      const uint4 a = ld_global_v4(src + (v << 4)), b = ld_global_v4(src + ((v + nth) << 4));
      const uint4 c = ld_global_v4(src + ((v + 2 * nth) << 4)), d = ld_global_v4(src + ((v + 3 * nth) << 4));
      multimem_st_v4(mc_dst + (v << 4), a);
      multimem_st_v4(mc_dst + ((v + nth) << 4), b);
      multimem_st_v4(mc_dst + ((v + 2 * nth) << 4), c);
      multimem_st_v4(mc_dst + ((v + 3 * nth) << 4), d);
    }
    for (; v < nvec; v += nth) multimem_st_v4(mc_dst + (v << 4), ld_global_v4(src + (v << 4)));
  }
}

int launch_multimem_bcast(void* mc_dst, const void* src, long long nbytes, int ctas, int threads, int iters,
                          cudaStream_t st) {
  if (mc_dst == nullptr || nbytes <= 0 || nbytes % 16 || ctas <= 0 || threads <= 0 || threads > 1024 || iters <= 0)
    return 1;
  if ((reinterpret_cast<uintptr_t>(mc_dst) | reinterpret_cast<uintptr_t>(src)) % 16) return 1;
  multimem_bcast_kernel<<<ctas, threads, 0, st>>>(static_cast<char*>(mc_dst), static_cast<const char*>(src), nbytes, iters);
  return 0;
}

}  // namespace b200ep
