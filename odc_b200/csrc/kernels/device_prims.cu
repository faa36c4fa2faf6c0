// Small kernels that exercise the device-side communication primitives one at a time (block put / get
// through a peer mapping, scalar put / get, atomic swap and compare-and-swap, the bounded grid barrier).
// They play the role of the reference's per-wrapper loop-back tests (tests/nvshmem_triton/test_putmem.py,
// test_getmem.py, test_atomic.py, test_p.py, test_g.py, test_utils.py) for this package's primitives.
#include "api.h"
#include "odc_device.cuh"

namespace odc {
namespace {

// copy `bytes` (multiple of 16) from src to dst with the whole block; either side may be a peer mapping
__device__ __forceinline__ void block_copy_16(void* dst, const void* src, size_t bytes) {
  const size_t nvec = bytes / 16;
  for (size_t v = threadIdx.x; v < nvec; v += blockDim.x)
    st_stream_v4(static_cast<uint4*>(dst) + v, ld_stream_v4(static_cast<const uint4*>(src) + v));
}

__global__ void put_block_kernel(void* remote_dst, const void* local_src, size_t bytes) {
  block_copy_16(remote_dst, local_src, bytes);
  __threadfence_system();
}

__global__ void get_block_kernel(void* local_dst, const void* remote_src, size_t bytes) {
  block_copy_16(local_dst, remote_src, bytes);
}

__global__ void scalar_put_get_kernel(int* remote_word, int value, int* readback) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(remote_word), "r"(value) : "memory");
    __threadfence_system();
    int v;
    asm volatile("ld.relaxed.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(remote_word) : "memory");
    *readback = v;
  }
}

// every CTA tries to claim the word: exactly one CAS sees the old value; swaps return what they displaced
__global__ void atomic_kernel(int* word, int* cas_seen, int* swap_seen, int expected_old, int cas_new, int swap_new) {
  if (threadIdx.x == 0) {
    cas_seen[blockIdx.x] = atomicCAS_system(word, expected_old, cas_new);
    swap_seen[blockIdx.x] = atomicExch_system(word + 1, swap_new);
  }
}

// all CTAs write their slot, meet at the barrier, then read their neighbour's slot
__global__ void grid_barrier_kernel(unsigned int* counter, int* slots, int* out, unsigned long long budget_ns,
                                    int* status) {
  if (threadIdx.x == 0) slots[blockIdx.x] = 1000 + blockIdx.x;
  const bool ok = grid_barrier_bounded(counter, gridDim.x, budget_ns, status);
  if (threadIdx.x == 0) out[blockIdx.x] = ok ? slots[(blockIdx.x + 1) % gridDim.x] : -1;
}

}  // namespace

cudaError_t launch_put_block(void* remote_dst, const void* local_src, size_t bytes, cudaStream_t s) {
  put_block_kernel<<<1, 1024, 0, s>>>(remote_dst, local_src, bytes);
  return cudaGetLastError();
}
cudaError_t launch_get_block(void* local_dst, const void* remote_src, size_t bytes, cudaStream_t s) {
  get_block_kernel<<<1, 1024, 0, s>>>(local_dst, remote_src, bytes);
  return cudaGetLastError();
}
cudaError_t launch_scalar_put_get(int* remote_word, int value, int* readback, cudaStream_t s) {
  scalar_put_get_kernel<<<1, 32, 0, s>>>(remote_word, value, readback);
  return cudaGetLastError();
}
cudaError_t launch_atomic_test(int* word, int* cas_seen, int* swap_seen, int ctas, int expected_old, int cas_new,
                               int swap_new, cudaStream_t s) {
  atomic_kernel<<<ctas, 32, 0, s>>>(word, cas_seen, swap_seen, expected_old, cas_new, swap_new);
  return cudaGetLastError();
}
cudaError_t launch_grid_barrier_test(unsigned int* counter, int* slots, int* out, int ctas,
                                     unsigned long long budget_ns, int* status, cudaStream_t s) {
  // all CTAs must be co-resident: the caller keeps ctas <= number of SMs
  grid_barrier_kernel<<<ctas, 64, 0, s>>>(counter, slots, out, budget_ns, status);
  return cudaGetLastError();
}

}  // namespace odc
