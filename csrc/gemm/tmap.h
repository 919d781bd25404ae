// Host helper: 2-D bf16 TMA tensor maps (128-byte swizzle) through the driver entry point that
// the CUDA runtime hands out, so the extension needs no link-time dependency on a driver stub.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

namespace b200ep {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled is a DRIVER entry point: it needs a CUDA context that is current on the
// calling thread. The runtime binds the primary context to a thread lazily, on the first runtime
// call that needs it, and worker threads (autograd's backward threads, any user thread) may reach
// the grouped GEMM launchers before they have made one: the encode then fails or crashes.
// cudaSetDevice on the thread's current device binds the context; done once per thread.
inline void tmap_bind_context_to_this_thread() {
  static thread_local bool bound = false;
  if (bound) return;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && cudaSetDevice(dev) == cudaSuccess) bound = true;
}

inline EncodeTiledFn tmap_encode_fn() {
  tmap_bind_context_to_this_thread();
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// bf16 tensor [rows, cols] (cols contiguous, this GPU's memory); box = box_cols x box_rows with
// box_cols * 2 == 128 bytes (one swizzle row). Reads outside the tensor return zeros.
// Returns 0 on success, 1 if the entry point is missing, 2 if the driver rejects the arguments.
inline int make_tmap_bf16(CUtensorMap* m, const void* base, long long rows, long long cols, int box_cols, int box_rows) {
  EncodeTiledFn fn = tmap_encode_fn();
  if (!fn) return 1;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 2;
}

}  // namespace b200ep
