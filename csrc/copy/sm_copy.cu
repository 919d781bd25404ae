// SM-driven peer copy kernels (the measured "LSU" and "TMA-staged" variants).
//
// Capability parity with the reference's four inline kernels
// (`LSU_TMA/nvlink_lsu_tma_copy_test.py:182-276`,
//  `LSU_TMA/nvlink_lsu_tma_round_robin_copy_test.py:291-406`), re-designed for B200:
//  * lsu_copy      : grid-stride 16-byte or 32-byte vector ld/st; either pointer may be a
//                    peer's memory (push or pull); optional persistent iteration loop.
//  * tma_staged    : a multi-stage shared-memory pipeline. Push: one elected thread streams
//                    LOCAL source tiles into shared memory with bulk async copies (mbarrier
//                    completion) while the consumer warps drain finished stages to the peer
//                    with 16-byte LSU stores. Pull: consumer warps fill stages with LSU peer
//                    loads and the elected thread writes them to LOCAL memory with bulk async
//                    stores. The bulk engine never touches another GPU's memory, and loads
//                    and stores overlap (the reference's kernel was single-buffered).
//  * round-robin   : both variants with a destination table; chunk c of the source goes to
//                    table[c % n_dst] at the same byte offset.
#include "../common.cuh"
#include "copy_api.h"

namespace b200ep {

// ---------------------------------------------------------------------------------------
// LSU copy
// ---------------------------------------------------------------------------------------
template <int VEC>  // 16 or 32 bytes per access; 1 = byte fallback
__global__ void lsu_copy_kernel(char* __restrict__ dst, const char* __restrict__ src,
                                long long nbytes, int iters) {
  // When launched with programmatic stream serialisation the next launch in the stream may
  // start as soon as every CTA has passed this point (independent copies need no further wait).
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  for (int it = 0; it < iters; ++it) {
    if (VEC == 1) {
      for (long long i = tid; i < nbytes; i += nth) dst[i] = src[i];
    } else {
      const long long nvec = nbytes / VEC;
      // 4 independent accesses in flight per thread.
      long long v = tid;
      for (; v + 3 * nth < nvec; v += 4 * nth) {
        if (VEC == 16) {
          uint4 a = ld_global_v4(src + v * 16), b = ld_global_v4(src + (v + nth) * 16);
          uint4 c = ld_global_v4(src + (v + 2 * nth) * 16), d = ld_global_v4(src + (v + 3 * nth) * 16);
          st_global_v4(dst + v * 16, a);
          st_global_v4(dst + (v + nth) * 16, b);
          st_global_v4(dst + (v + 2 * nth) * 16, c);
          st_global_v4(dst + (v + 3 * nth) * 16, d);
        } else {
          u32x8 a = ld_global_v8(src + v * 32), b = ld_global_v8(src + (v + nth) * 32);
          u32x8 c = ld_global_v8(src + (v + 2 * nth) * 32), d = ld_global_v8(src + (v + 3 * nth) * 32);
          st_global_v8(dst + v * 32, a);
          st_global_v8(dst + (v + nth) * 32, b);
          st_global_v8(dst + (v + 2 * nth) * 32, c);
          st_global_v8(dst + (v + 3 * nth) * 32, d);
        }
      }
      for (; v < nvec; v += nth) {
        if (VEC == 16) st_global_v4(dst + v * 16, ld_global_v4(src + v * 16));
        else st_global_v8(dst + v * 32, ld_global_v8(src + v * 32));
      }
      for (long long i = nvec * VEC + tid; i < nbytes; i += nth) dst[i] = src[i];
    }
  }
}

template <int VEC>
static void lsu_launch(char* d, const char* s, long long nbytes, int ctas, int threads, int iters, bool overlap,
                       cudaStream_t st) {
  if (!overlap) {
    lsu_copy_kernel<VEC><<<ctas, threads, 0, st>>>(d, s, nbytes, iters);
    return;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ctas);
  cfg.blockDim = dim3(threads);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, lsu_copy_kernel<VEC>, d, s, nbytes, iters);
}

// vec_bytes: 16 or 32; add 256 to let consecutive launches in the stream overlap (programmatic
// dependent launch): meant for back-to-back INDEPENDENT copies, where the launch latency and the
// drain of the previous kernel otherwise dominate small messages.
int launch_lsu_copy(void* dst, const void* src, long long nbytes, int ctas, int threads,
                    int iters, int vec_bytes, cudaStream_t st) {
  if (nbytes <= 0 || ctas <= 0 || threads <= 0 || threads > 1024 || iters <= 0) return 1;
  const bool overlap = (vec_bytes & 256) != 0;
  vec_bytes &= 255;
  const uintptr_t a = reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src);
  char* d = static_cast<char*>(dst);
  const char* s = static_cast<const char*>(src);
  if (vec_bytes == 32 && (a % 32) == 0)
    lsu_launch<32>(d, s, nbytes, ctas, threads, iters, overlap, st);
  else if (vec_bytes >= 16 && (a % 16) == 0)
    lsu_launch<16>(d, s, nbytes, ctas, threads, iters, overlap, st);
  else
    lsu_launch<1>(d, s, nbytes, ctas, threads, iters, overlap, st);
  return 0;
}

// Round-robin LSU copy: 16-byte vectors, destination chosen per chunk.
struct DstTable { char* p[kMaxRanks]; int n; };

__global__ void lsu_rr_copy_kernel(DstTable tab, const char* __restrict__ src, long long nbytes,
                                   long long rr_bytes, int iters, int aligned) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  for (int it = 0; it < iters; ++it) {
    if (aligned) {
      const long long nvec = nbytes >> 4;
      for (long long v = tid; v < nvec; v += nth) {
        const long long off = v << 4;
        char* d = tab.p[(off / rr_bytes) % tab.n];
        st_global_v4(d + off, ld_global_v4(src + off));
      }
    } else {
      for (long long i = tid; i < nbytes; i += nth) tab.p[(i / rr_bytes) % tab.n][i] = src[i];
    }
  }
}

int launch_lsu_rr_copy(void* const* dsts, int n_dst, const void* src, long long nbytes,
                       long long rr_bytes, int ctas, int threads, int iters, cudaStream_t st) {
  if (n_dst <= 0 || n_dst > kMaxRanks || nbytes <= 0 || rr_bytes <= 0 || ctas <= 0 ||
      threads <= 0 || threads > 1024 || iters <= 0)
    return 1;
  DstTable tab;
  tab.n = n_dst;
  uintptr_t a = reinterpret_cast<uintptr_t>(src) | (uintptr_t)nbytes | (uintptr_t)rr_bytes;
  for (int i = 0; i < n_dst; ++i) {
    tab.p[i] = static_cast<char*>(dsts[i]);
    a |= reinterpret_cast<uintptr_t>(dsts[i]);
  }
  lsu_rr_copy_kernel<<<ctas, threads, 0, st>>>(tab, static_cast<const char*>(src), nbytes,
                                               rr_bytes, iters, (a % 16) == 0 ? 1 : 0);
  return 0;
}

// ---------------------------------------------------------------------------------------
// mbarrier / bulk-copy primitives (local memory only)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait; false after ~2 s (records kTimeoutMbarrier).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* status) {
  if (mbar_try(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 0; it < (1u << 30); ++it) {
    if (mbar_try(bar, parity)) return true;
    if ((it & 255) == 255 && globaltimer_ns() - t0 > 2000000000ull) break;
  }
  set_status(status, kTimeoutMbarrier);
  return false;
}
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_s2g(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

constexpr int kMaxStages = 8;

// Work decomposition shared by the staged kernels: the byte range is cut into tiles of
// `tile` bytes; CTA b owns tiles b, b+grid, ... ; for round-robin each tile is further cut at
// rr-chunk boundaries so that one piece never spans two destinations.
struct StagedArgs {
  const char* src;     // push: local; pull: peer
  DstTable dst;        // push: peer(s); pull: n = 1, local
  long long nbytes;
  long long rr_bytes;  // 0 = single destination
  int tile;            // bytes per stage (multiple of 16)
  int piece;           // bytes per bulk store in pull mode (multiple of 16, <= tile)
  int stages;
  int iters;
  int* status;
};

__device__ __forceinline__ char* rr_dst(const DstTable& t, long long off, long long rr_bytes) {
  return rr_bytes > 0 ? t.p[(off / rr_bytes) % t.n] : t.p[0];
}

// PUSH: bulk loads local src -> smem; consumer warps store smem -> peer(s) with LSU.
__global__ void tma_staged_push_kernel(StagedArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full[kMaxStages], empty[kMaxStages];
  __shared__ int abort_flag;
  const int ncons = blockDim.x - 32;  // warp 0 is the producer warp
  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], ncons / 32); }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const long long ntiles = (a.nbytes + a.tile - 1) / a.tile;
  const long long my_tiles = blockIdx.x < ntiles ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const long long total = my_tiles * a.iters;
  if (threadIdx.x == 0) {
    long long issued = 0;
    for (long long n = 0; n < total; ++n) {
      const int s = n % a.stages;
      const uint32_t ph = (n / a.stages) & 1;
      if (n >= a.stages && !mbar_wait(&empty[s], ph ^ 1, a.status)) { abort_flag = 1; break; }
      if (*(volatile int*)&abort_flag) break;
      const long long tile_idx = blockIdx.x + (n % my_tiles) * gridDim.x;
      const long long off = tile_idx * a.tile;
      const uint32_t bytes = (uint32_t)min((long long)a.tile, a.nbytes - off);
      mbar_expect_tx(&full[s], bytes);
      bulk_g2s(smem + (size_t)s * a.tile, a.src + off, bytes, &full[s]);
      issued = n + 1;
    }
    if (*(volatile int*)&abort_flag) {
      // Let our own loads in flight land before the CTA's shared memory is released.
      for (long long n = (issued > a.stages ? issued - a.stages : 0); n < issued; ++n)
        mbar_wait(&full[n % a.stages], (n / a.stages) & 1, nullptr);
    }
  } else if (threadIdx.x >= 32) {
    const int ct = threadIdx.x - 32;
    for (long long n = 0; n < total; ++n) {
      const int s = n % a.stages;
      const uint32_t ph = (n / a.stages) & 1;
      if (*(volatile int*)&abort_flag) break;
      if (!mbar_wait(&full[s], ph, a.status)) { abort_flag = 1; break; }
      const long long tile_idx = blockIdx.x + (n % my_tiles) * gridDim.x;
      const long long off = tile_idx * a.tile;
      const int bytes = (int)min((long long)a.tile, a.nbytes - off);
      const unsigned char* sp = smem + (size_t)s * a.tile;
      for (int v = ct * 16; v < bytes; v += ncons * 16) {
        const uint4 val = *reinterpret_cast<const uint4*>(sp + v);
        st_global_v4(rr_dst(a.dst, off + v, a.rr_bytes) + off + v, val);
      }
      __syncwarp();
      if ((threadIdx.x & 31) == 0) mbar_arrive(&empty[s]);
    }
  }
}

// PULL: consumer warps load peer src -> smem with LSU; the elected thread bulk-stores
// finished stages into LOCAL dst in `piece`-sized copies.
__global__ void tma_staged_pull_kernel(StagedArgs a) {
  extern __shared__ __align__(128) unsigned char smem[];
  __shared__ uint64_t full[kMaxStages], empty[kMaxStages];
  __shared__ int abort_flag;
  const int nload = blockDim.x - 32;
  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) { mbar_init(&full[s], nload / 32); mbar_init(&empty[s], 1); }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const long long ntiles = (a.nbytes + a.tile - 1) / a.tile;
  const long long my_tiles = blockIdx.x < ntiles ? (ntiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const long long total = my_tiles * a.iters;
  if (threadIdx.x == 0) {
    for (long long n = 0; n < total; ++n) {
      const int s = n % a.stages;
      const uint32_t ph = (n / a.stages) & 1;
      if (*(volatile int*)&abort_flag) break;
      if (!mbar_wait(&full[s], ph, a.status)) { abort_flag = 1; break; }
      const long long tile_idx = blockIdx.x + (n % my_tiles) * gridDim.x;
      const long long off = tile_idx * a.tile;
      const int bytes = (int)min((long long)a.tile, a.nbytes - off);
      fence_proxy_async_smem();
      for (int p = 0; p < bytes; p += a.piece)
        bulk_s2g(a.dst.p[0] + off + p, smem + (size_t)s * a.tile + p, (uint32_t)min(a.piece, bytes - p));
      bulk_commit();
      bulk_wait_read<0>();  // smem of this stage may be refilled once the engine has read it
      mbar_arrive(&empty[s]);
    }
    bulk_wait_all();
  } else if (threadIdx.x >= 32) {
    const int ct = threadIdx.x - 32;
    for (long long n = 0; n < total; ++n) {
      const int s = n % a.stages;
      const uint32_t ph = (n / a.stages) & 1;
      if (*(volatile int*)&abort_flag) break;
      if (n >= a.stages && !mbar_wait(&empty[s], ph ^ 1, a.status)) { abort_flag = 1; break; }
      const long long tile_idx = blockIdx.x + (n % my_tiles) * gridDim.x;
      const long long off = tile_idx * a.tile;
      const int bytes = (int)min((long long)a.tile, a.nbytes - off);
      unsigned char* sp = smem + (size_t)s * a.tile;
      for (int v = ct * 16; v < bytes; v += nload * 16)
        *reinterpret_cast<uint4*>(sp + v) = ld_global_v4(a.src + off + v);
      fence_proxy_async_smem();
      __syncwarp();
      if ((threadIdx.x & 31) == 0) mbar_arrive(&full[s]);
    }
  }
}

static int staged_check(const void* src, long long nbytes, int tile, int piece, int stages,
                        int ctas, int threads, int iters, long long rr_bytes) {
  if (nbytes <= 0 || nbytes % 16 || tile <= 0 || tile % 16 || piece <= 0 || piece % 16) return 1;
  if (piece > tile || stages < 1 || stages > kMaxStages || ctas <= 0 || iters <= 0) return 1;
  if (threads < 64 || threads > 1024 || threads % 32) return 1;
  if (reinterpret_cast<uintptr_t>(src) % 16) return 1;
  if (rr_bytes < 0 || rr_bytes % 16) return 1;
  return 0;
}

int launch_tma_staged_copy(void* const* dsts, int n_dst, const void* src, long long nbytes,
                           long long rr_bytes, int pull, int tile, int piece, int stages, int ctas,
                           int threads, int iters, int* status, cudaStream_t st) {
  if (n_dst <= 0 || n_dst > kMaxRanks) return 1;
  if (staged_check(src, nbytes, tile, piece, stages, ctas, threads, iters, rr_bytes)) return 1;
  if (pull && (n_dst != 1 || rr_bytes != 0)) return 1;
  StagedArgs a;
  a.src = static_cast<const char*>(src);
  a.dst.n = n_dst;
  for (int i = 0; i < n_dst; ++i) {
    if (reinterpret_cast<uintptr_t>(dsts[i]) % 16) return 1;
    a.dst.p[i] = static_cast<char*>(dsts[i]);
  }
  a.nbytes = nbytes; a.rr_bytes = rr_bytes; a.tile = tile; a.piece = piece;
  a.stages = stages; a.iters = iters; a.status = status;
  const size_t smem = (size_t)tile * stages;
  auto kern = pull ? tma_staged_pull_kernel : tma_staged_push_kernel;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return 2;
  }
  kern<<<ctas, threads, smem, st>>>(a);
  return 0;
}

}  // namespace b200ep
