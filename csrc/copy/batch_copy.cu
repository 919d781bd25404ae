// One-launch table of copies: the SM counterpart of a batched memcpy submission
// (the reference submits N copies with one runtime call,
// `Copy_Engine/nvlink_copy_engine_test.py:281-304`; here one kernel launch covers N
// descriptors, each served by `ctas_per_copy` CTAs with 16-byte vector ld/st).
#include "../common.cuh"
#include "copy_api.h"

namespace b200ep {

__global__ void batched_copy_kernel(const CopyDesc* __restrict__ desc, int n) {
  const int c = blockIdx.y;
  if (c >= n) return;
  const CopyDesc d = desc[c];
  char* dst = static_cast<char*>(d.dst);
  const char* src = static_cast<const char*>(d.src);
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src)) & 15) == 0;
  if (aligned) {
    const long long nvec = d.nbytes >> 4;
    long long v = tid;
    for (; v + nth < nvec; v += 2 * nth) {
      const uint4 a = ld_global_v4(src + (v << 4)), b = ld_global_v4(src + ((v + nth) << 4));
      st_global_v4(dst + (v << 4), a);
      st_global_v4(dst + ((v + nth) << 4), b);
    }
    for (; v < nvec; v += nth) st_global_v4(dst + (v << 4), ld_global_v4(src + (v << 4)));
    for (long long i = (nvec << 4) + tid; i < d.nbytes; i += nth) dst[i] = src[i];
  } else {
    for (long long i = tid; i < d.nbytes; i += nth) dst[i] = src[i];
  }
}

int launch_batched_copy(const CopyDesc* desc_dev, int n, int ctas_per_copy, int threads,
                        cudaStream_t st) {
  if (n <= 0 || n > 65535 || ctas_per_copy <= 0 || threads <= 0 || threads > 1024) return 1;
  batched_copy_kernel<<<dim3(ctas_per_copy, n), threads, 0, st>>>(desc_dev, n);
  return 0;
}

}  // namespace b200ep
