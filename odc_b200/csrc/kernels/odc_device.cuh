// Device-side communication primitives over peer mappings: vector peer loads, remote vector
// reductions, system-scope release/acquire flags and bounded waits that report instead of hanging.
// Takes the role of the NVSHMEM device calls used by the reference's Triton kernels
// (odc/primitives/nvshmem_triton.py:131-277) and of its unbounded grid barrier
// (odc/primitives/utils.py:245-256).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace odc {

// status word layout: [0] error code, [1] detail, [2] observed value, [3] spare
enum StatusCode : int {
  kOk = 0,
  kErrWaitTimeout = 1,
  kErrBounds = 2,
  kErrPeerIndex = 3,
  kErrPipelineTimeout = 4,
};

__device__ __forceinline__ void report(int* status, int code, int detail, int seen) {
  if (status != nullptr && atomicCAS(status, 0, code) == 0) {
    status[1] = detail;
    status[2] = seen;
    __threadfence_system();
  }
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// 16-byte load that does not pollute L1 (peer or local global memory).
__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ void st_stream_v4(void* p, uint4 v) {
  asm volatile("st.global.L1::no_allocate.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}

// Remote (or local) fp32 vector reduction, relaxed, system scope: 16 bytes per instruction.
__device__ __forceinline__ void red_add_v4_f32(float* p, float a, float b, float c, float d) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

__device__ __forceinline__ void red_add_f32(float* p, float a) {
  asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(p), "f"(a) : "memory");
}

__device__ __forceinline__ void red_add_bf16x2(void* p, uint32_t packed) {
  asm volatile("red.relaxed.sys.global.add.noftz.bf16x2 [%0], %1;" ::"l"(p), "r"(packed) : "memory");
}

// Arrival signal: everything this thread has observed (including other threads' writes ordered
// before it by a barrier + fence) becomes visible to whoever acquires the counter.
__device__ __forceinline__ void signal_add_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}

// Spin until *p >= target or the budget runs out.  Returns true on success.  On timeout the
// status word is written and the caller returns normally: the context stays usable.
__device__ __forceinline__ bool bounded_wait_ge(const unsigned long long* p, unsigned long long target,
                                                uint64_t budget_ns, int* status, int detail) {
  uint64_t t0 = globaltimer_ns();
  unsigned long long v = ld_acquire_sys(p);
  while (v < target) {
    __nanosleep(256);
    if (globaltimer_ns() - t0 > budget_ns) {
      report(status, kErrWaitTimeout, detail, static_cast<int>(v));
      return false;
    }
    v = ld_acquire_sys(p);
  }
  return true;
}

// Grid-wide barrier on a monotonic counter (the caller passes the same zero-initialised word to every
// launch that uses it only once, or tracks the running target itself).  All CTAs of the grid must be
// co-resident.  Bounded: on timeout the status word is written and false is returned to every thread.
__device__ __forceinline__ bool grid_barrier_bounded(unsigned int* counter, unsigned int expected,
                                                     uint64_t budget_ns, int* status) {
  __shared__ int ok_flag;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(counter, 1u);
    const uint64_t t0 = globaltimer_ns();
    ok_flag = 1;
    unsigned int v;
    while (true) {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
      if (v >= expected) break;
      if (globaltimer_ns() - t0 > budget_ns) {
        report(status, kErrWaitTimeout, 1, static_cast<int>(v));
        ok_flag = 0;
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return ok_flag != 0;
}

}  // namespace odc
