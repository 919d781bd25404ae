// Shared device helpers for every sm_100a kernel in this library: status words,
// bounded waits, system-scope release/acquire flags, vector ld/st on peer memory.
//
// Design rules that the helpers encode:
//  * Cross-GPU bytes move only by LSU loads/stores on peer-mapped pointers
//    (or multimem); TMA is used on this GPU's own memory only.
//  * No wait is unbounded. A wait that runs out records a code in a status
//    block and returns false; callers then skip the dependent work and return, so
//    the context stays usable. The status block is device memory (word 0 = first
//    code recorded); words 2-3 may hold the device-visible address of a pinned
//    host word that receives a copy of the code, so that the host can notice a
//    fault without synchronising the device.
//  * Flags are monotonically increasing epochs, never reset: a waiter waits for
//    flag >= epoch. Payload regions are double-buffered by epoch parity, which
//    makes a start-of-op barrier unnecessary (a rank can never run two epochs
//    ahead of a peer because each op ends by waiting for every peer's flag).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200ep {

constexpr int kMaxRanks = 16;

// Status codes written to the status word (first error wins).
enum Status : int {
  kOk = 0,
  kTimeoutNotify = 1,     // peers' token counts did not arrive in time
  kTimeoutDispatch = 2,   // peers' dispatch-done flags did not arrive
  kTimeoutCombine = 3,    // peers' combine-done flags did not arrive
  kTimeoutLowLatency = 4, // low-latency per-expert counts did not arrive
  kTimeoutBarrier = 5,
  kOverflowRecv = 6,      // a receive row index exceeded the buffer capacity
  kBadExpertIndex = 7,    // topk_idx outside [-1, num_experts)
  kTimeoutProbe = 8,      // the self-test wait (flag nobody sets) ran out, as intended
  kTimeoutMbarrier = 9,   // a TMA/MMA mbarrier wait inside a kernel ran out
  kOverflowSlots = 10,
};

struct PeerPtrs {
  // Base address of every rank's symmetric region, as mapped in THIS process.
  char* base[kMaxRanks];
};

// Cumulative 32-bit counters (low-latency arrival counters) are compared modulo 2^32:
// `have` has reached `want` when it is at most 2^31 - 1 increments ahead of it. A signed
// `have >= want` would turn false->true at the 0x7fffffff -> 0x80000000 wrap of `want`.
#if defined(__CUDACC__)
__host__ __device__
#endif
inline bool counter_reached(uint32_t have, uint32_t want) {
  return static_cast<int32_t>(have - want) >= 0;
}

#ifdef __CUDACC__
__device__ __forceinline__ void set_status(int* status, int code) {
  if (status == nullptr) return;
  if (atomicCAS_system(status, 0, code) == 0) {
    // first error of this block: mirror it to the host word, if one is registered
    int* host = *reinterpret_cast<int* volatile*>(status + 2);
    if (host != nullptr) *reinterpret_cast<volatile int*>(host) = code;
  }
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_relaxed_sys(const int* p) {
  int v;
  asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}

// Wait until *flag >= want, at most timeout_ns nanoseconds. Returns true on success.
// On time-out records `code` in the status word and returns false.
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int want, uint64_t timeout_ns,
                                             int* status, int code) {
  if (ld_acquire_sys(flag) >= want) return true;
  const uint64_t t0 = globaltimer_ns();
  // The iteration cap bounds the loop even if the timer misbehaves.
  for (uint64_t it = 0; it < (1ull << 34); ++it) {
    if (ld_acquire_sys(flag) >= want) return true;
    if ((it & 63) == 63 && globaltimer_ns() - t0 > timeout_ns) break;
    __nanosleep(32);
  }
  set_status(status, code);
  return false;
}

// Same bounded wait for a cumulative counter that may wrap around 2^32.
__device__ __forceinline__ bool wait_counter_reached(const int* flag, uint32_t want, uint64_t timeout_ns,
                                                     int* status, int code) {
  if (counter_reached((uint32_t)ld_acquire_sys(flag), want)) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint64_t it = 0; it < (1ull << 34); ++it) {
    if (counter_reached((uint32_t)ld_acquire_sys(flag), want)) return true;
    if ((it & 63) == 63 && globaltimer_ns() - t0 > timeout_ns) break;
    __nanosleep(32);
  }
  set_status(status, code);
  return false;
}

// 16-byte vector access. Peer stores bypass L1 allocation; streaming local loads use
// the non-coherent path only where the data is read-only for the kernel's lifetime.
__device__ __forceinline__ uint4 ld_global_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ld_global_nc_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_global_v4(void* p, const uint4& v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};"
               ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// 32-byte vector access (sm_100+ only).
struct __align__(32) u32x8 { uint32_t v[8]; };
__device__ __forceinline__ u32x8 ld_global_v8(const void* p) {
  u32x8 r;
  asm volatile("ld.global.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]),
                 "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]), "=r"(r.v[7]) : "l"(p));
  return r;
}
__device__ __forceinline__ void st_global_v8(void* p, const u32x8& r) {
  asm volatile("st.global.v8.u32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"l"(p), "r"(r.v[0]), "r"(r.v[1]), "r"(r.v[2]), "r"(r.v[3]),
                 "r"(r.v[4]), "r"(r.v[5]), "r"(r.v[6]), "r"(r.v[7]) : "memory");
}

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// "Last block done" bookkeeping: every block calls this once after its work; exactly one
// caller (the last) gets true, and all earlier blocks' global writes are visible to it.
__device__ __forceinline__ bool last_block_arrive(unsigned int* counter, unsigned int nblocks) {
  __shared__ bool is_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_acq_rel_sys();
    unsigned int prev = atomicAdd(counter, 1u);
    is_last = (prev == nblocks - 1);
    // The last block only needs to ACQUIRE what the others published on this GPU (they made
    // their own peer stores system-visible before arriving); its later flag stores are releases.
    if (is_last) { *counter = 0; asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
  }
  __syncthreads();
  return is_last;
}

#endif  // __CUDACC__

}  // namespace b200ep
