// SwiGLU x routing-probability, forward and backward, for the training path of the expert MLP
// (the inference path fuses the forward into the fc1 GEMM epilogue instead).
//   h = [gate | linear]  (bf16 [rows, 2F]),  act = silu(gate) * linear * p[row]
// Backward, given dact:  dp[row] = sum_f dact * silu(gate) * linear
//                         dlinear = dact * p * silu(gate)
//                         dgate   = dact * p * linear * sig(gate) * (1 + gate * (1 - sig(gate)))
// One CTA per row, 16-byte accesses. Replaces the separate activation / multiply / cast kernels of
// `DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:539-540,597-598` and their autograd twins.
#include <cuda_bf16.h>
#include "../common.cuh"
#include "gemm_api.h"

namespace b200ep {

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) { f[2 * q] = __uint_as_float(u[q] << 16); f[2 * q + 1] = __uint_as_float(u[q] & 0xffff0000u); }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 o;
  uint32_t* u = &o.x;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * q], f[2 * q + 1]);
    u[q] = *reinterpret_cast<uint32_t*>(&h);
  }
  return o;
}

__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const char* __restrict__ h, const float* __restrict__ p, char* __restrict__ act,
                  const int* __restrict__ n_rows_ptr, int max_rows, int F) {
  const int rows = n_rows_ptr ? min(*n_rows_ptr, max_rows) : max_rows;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const float pr = p ? p[r] : 1.f;
    const char* g = h + (size_t)r * F * 4;          // 2F bf16 per row
    const char* l = g + (size_t)F * 2;
    char* o = act + (size_t)r * F * 2;
    for (int v = threadIdx.x; v < F / 8; v += blockDim.x) {
      float fg[8], fl[8], fo[8];
      unpack8(ld_global_nc_v4(g + ((size_t)v << 4)), fg);
      unpack8(ld_global_nc_v4(l + ((size_t)v << 4)), fl);
#pragma unroll
      for (int i = 0; i < 8; ++i) fo[i] = fg[i] / (1.f + __expf(-fg[i])) * fl[i] * pr;
      st_global_v4(o + ((size_t)v << 4), pack8(fo));
    }
  }
}

__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const char* __restrict__ h, const float* __restrict__ p, const char* __restrict__ dact,
                  char* __restrict__ dh, float* __restrict__ dp, const int* __restrict__ n_rows_ptr,
                  int max_rows, int F) {
  __shared__ float s_part[8];
  const int rows = n_rows_ptr ? min(*n_rows_ptr, max_rows) : max_rows;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const float pr = p ? p[r] : 1.f;
    const char* g = h + (size_t)r * F * 4;
    const char* l = g + (size_t)F * 2;
    const char* d = dact + (size_t)r * F * 2;
    char* og = dh + (size_t)r * F * 4;
    char* ol = og + (size_t)F * 2;
    float acc = 0.f;
    for (int v = threadIdx.x; v < F / 8; v += blockDim.x) {
      float fg[8], fl[8], fd[8], dg[8], dl[8];
      unpack8(ld_global_nc_v4(g + ((size_t)v << 4)), fg);
      unpack8(ld_global_nc_v4(l + ((size_t)v << 4)), fl);
      unpack8(ld_global_nc_v4(d + ((size_t)v << 4)), fd);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float sig = 1.f / (1.f + __expf(-fg[i]));
        const float s = fg[i] * sig;
        acc += fd[i] * s * fl[i];
        const float da = fd[i] * pr;
        dl[i] = da * s;
        dg[i] = da * fl[i] * sig * (1.f + fg[i] * (1.f - sig));
      }
      st_global_v4(og + ((size_t)v << 4), pack8(dg));
      st_global_v4(ol + ((size_t)v << 4), pack8(dl));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0 && dp != nullptr) {
      float t = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += s_part[w];
      dp[r] = t;
    }
    __syncthreads();
  }
}

int launch_swiglu_fwd(const void* h, const float* p, void* act, const int* n_rows_ptr, int max_rows, int F,
                      cudaStream_t st) {
  if (F <= 0 || F % 8 || max_rows < 0) return 1;
  if (max_rows == 0) return 0;
  swiglu_fwd_kernel<<<min(max_rows, 148 * 16), 256, 0, st>>>(static_cast<const char*>(h), p, static_cast<char*>(act),
                                                             n_rows_ptr, max_rows, F);
  return 0;
}

int launch_swiglu_bwd(const void* h, const float* p, const void* dact, void* dh, float* dp, const int* n_rows_ptr,
                      int max_rows, int F, cudaStream_t st) {
  if (F <= 0 || F % 8 || max_rows < 0) return 1;
  if (max_rows == 0) return 0;
  swiglu_bwd_kernel<<<min(max_rows, 148 * 16), 256, 0, st>>>(static_cast<const char*>(h), p, static_cast<const char*>(dact),
                                                             static_cast<char*>(dh), dp, n_rows_ptr, max_rows, F);
  return 0;
}

// ---------------------------------------------------------------------------------------
// Ungated activations (gelu / silu / relu) x routing probability, forward and backward:
//   act = f(h) * p[row],   dh = dact * p * f'(h),   dp[row] = sum_f dact * f(h)
// kind: 0 gelu (erf form, as torch.nn.functional.gelu), 1 silu, 2 relu.
// (`DeepEP_Megatron/test_deepep_moe_dispatch_combine.py:516-526` offers these beside swiglu.)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void act_eval(int kind, float x, float* f, float* df) {
  if (kind == 0) {
    const float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
    const float pdf = 0.39894228040143268f * __expf(-0.5f * x * x);
    *f = x * cdf;
    *df = cdf + x * pdf;
  } else if (kind == 1) {
    const float sig = 1.f / (1.f + __expf(-x));
    *f = x * sig;
    *df = sig * (1.f + x * (1.f - sig));
  } else {
    *f = x > 0.f ? x : 0.f;
    *df = x > 0.f ? 1.f : 0.f;
  }
}

__global__ void __launch_bounds__(256)
act_fwd_kernel(const char* __restrict__ h, const float* __restrict__ p, char* __restrict__ act,
               const int* __restrict__ n_rows_ptr, int max_rows, int F, int kind) {
  const int rows = n_rows_ptr ? min(*n_rows_ptr, max_rows) : max_rows;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const float pr = p ? p[r] : 1.f;
    const char* g = h + (size_t)r * F * 2;
    char* o = act + (size_t)r * F * 2;
    for (int v = threadIdx.x; v < F / 8; v += blockDim.x) {
      float fg[8], fo[8];
      unpack8(ld_global_nc_v4(g + ((size_t)v << 4)), fg);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float f, df;
        act_eval(kind, fg[i], &f, &df);
        fo[i] = f * pr;
      }
      st_global_v4(o + ((size_t)v << 4), pack8(fo));
    }
  }
}

__global__ void __launch_bounds__(256)
act_bwd_kernel(const char* __restrict__ h, const float* __restrict__ p, const char* __restrict__ dact,
               char* __restrict__ dh, float* __restrict__ dp, const int* __restrict__ n_rows_ptr,
               int max_rows, int F, int kind) {
  __shared__ float s_part[8];
  const int rows = n_rows_ptr ? min(*n_rows_ptr, max_rows) : max_rows;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const float pr = p ? p[r] : 1.f;
    const char* g = h + (size_t)r * F * 2;
    const char* d = dact + (size_t)r * F * 2;
    char* og = dh + (size_t)r * F * 2;
    float acc = 0.f;
    for (int v = threadIdx.x; v < F / 8; v += blockDim.x) {
      float fg[8], fd[8], dg[8];
      unpack8(ld_global_nc_v4(g + ((size_t)v << 4)), fg);
      unpack8(ld_global_nc_v4(d + ((size_t)v << 4)), fd);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float f, df;
        act_eval(kind, fg[i], &f, &df);
        acc += fd[i] * f;
        dg[i] = fd[i] * pr * df;
      }
      st_global_v4(og + ((size_t)v << 4), pack8(dg));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0 && dp != nullptr) {
      float t = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += s_part[w];
      dp[r] = t;
    }
    __syncthreads();
  }
}

int launch_act_fwd(const void* h, const float* p, void* act, const int* n_rows_ptr, int max_rows, int F, int kind,
                   cudaStream_t st) {
  if (F <= 0 || F % 8 || max_rows < 0 || kind < 0 || kind > 2) return 1;
  if (max_rows == 0) return 0;
  act_fwd_kernel<<<min(max_rows, 148 * 16), 256, 0, st>>>(static_cast<const char*>(h), p, static_cast<char*>(act),
                                                          n_rows_ptr, max_rows, F, kind);
  return 0;
}

int launch_act_bwd(const void* h, const float* p, const void* dact, void* dh, float* dp, const int* n_rows_ptr,
                   int max_rows, int F, int kind, cudaStream_t st) {
  if (F <= 0 || F % 8 || max_rows < 0 || kind < 0 || kind > 2) return 1;
  if (max_rows == 0) return 0;
  act_bwd_kernel<<<min(max_rows, 148 * 16), 256, 0, st>>>(static_cast<const char*>(h), p, static_cast<const char*>(dact),
                                                          static_cast<char*>(dh), dp, n_rows_ptr, max_rows, F, kind);
  return 0;
}

}  // namespace b200ep
