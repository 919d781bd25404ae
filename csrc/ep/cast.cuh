// bf16 -> fp8 e4m3 with one f32 scale per 128 channels ("1x128 block scaling").
// A warp converts 512 consecutive channels per step: each lane owns 16 channels, eight
// neighbouring lanes share one scale block. scale = max(amax, 1e-4) / 448.
#pragma once
#include <cuda_fp8.h>
#include "../common.cuh"

namespace b200ep {

__device__ __forceinline__ float bf16lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

__device__ __forceinline__ uint32_t cvt4_e4m3(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

// a, b: the lane's 16 bf16 values (two 16-byte vectors; zeros for inactive lanes).
// Must be called by all 32 lanes. Returns the 16 fp8 bytes; *scale is the block's scale.
__device__ __forceinline__ uint4 cast_block_fp8(const uint4& a, const uint4& b, float* scale) {
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  float f[16];
#pragma unroll
  for (int q = 0; q < 8; ++q) { f[2 * q] = bf16lo(w[q]); f[2 * q + 1] = bf16hi(w[q]); }
  float amax = 0.f;
#pragma unroll
  for (int q = 0; q < 16; ++q) amax = fmaxf(amax, fabsf(f[q]));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
  amax = fmaxf(amax, 1e-4f);
  *scale = amax * (1.f / 448.f);
  const float inv = 448.f / amax;
  uint4 o;
  o.x = cvt4_e4m3(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
  o.y = cvt4_e4m3(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
  o.z = cvt4_e4m3(f[8] * inv, f[9] * inv, f[10] * inv, f[11] * inv);
  o.w = cvt4_e4m3(f[12] * inv, f[13] * inv, f[14] * inv, f[15] * inv);
  return o;
}

}  // namespace b200ep
