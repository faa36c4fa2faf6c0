// See no_alloc.h.  Self-contained on purpose: the regular RMSNorm path is not touched.
#include "no_alloc.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

namespace {

constexpr int kThreads = 256;
constexpr int kMaxVec = 4;  // 256 threads x 8 bf16 x 4 = 8192 columns held in registers
constexpr int kMaxDevices = 64;

// The workspace: per-CTA partial sums of dw.  In host code this name is only a handle for the
// runtime (its host address is NOT device memory); host code must use the address obtained with
// cudaGetSymbolAddress below.
static __device__ __align__(256) float g_partials[ODC_NOALLOC_MAX_CTAS * ODC_NOALLOC_MAX_COLS];

float* g_partials_addr[kMaxDevices] = {nullptr};
std::mutex g_setup_mutex;

__device__ __forceinline__ float lo(unsigned u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float hi(unsigned u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  f[0] = lo(u.x); f[1] = hi(u.x); f[2] = lo(u.y); f[3] = hi(u.y);
  f[4] = lo(u.z); f[5] = hi(u.z); f[6] = lo(u.w); f[7] = hi(u.w);
}
__device__ __forceinline__ unsigned pack(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < kThreads / 32) ? red[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// dx = rstd * (dy*w - x * rstd^2 * mean(dy*w*x)); each CTA keeps its share of dw in registers and
// writes one row of the workspace (every column of that row, so stale contents never survive).
__global__ void __launch_bounds__(kThreads)
rmsnorm_bwd_noalloc_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                           const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                           __nv_bfloat16* __restrict__ dx, float* __restrict__ partials, int rows, int cols) {
  __shared__ float red[32];
  const int nvec = cols / 8;
  float dw[kMaxVec][8];
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k)
#pragma unroll
    for (int i = 0; i < 8; ++i) dw[k][i] = 0.f;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(row) * cols);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + size_t(row) * cols);
    const float rstd = rstd_in[row];
    uint4 xv[kMaxVec], gv[kMaxVec];
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxVec; ++k) {
      const int v = threadIdx.x + k * kThreads;
      if (v < nvec) {
        xv[k] = xr[v];
        gv[k] = gr[v];
        float xf[8], gf[8], wf[8];
        unpack8(xv[k], xf); unpack8(gv[k], gf); unpack8(wr[v], wf);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          dot += gf[i] * wf[i] * xf[i];
          dw[k][i] += gf[i] * xf[i] * rstd;
        }
      }
    }
    dot = block_sum(dot, red);
    const float c = dot * rstd * rstd / cols;
    uint4* dr = reinterpret_cast<uint4*>(dx + size_t(row) * cols);
#pragma unroll
    for (int k = 0; k < kMaxVec; ++k) {
      const int v = threadIdx.x + k * kThreads;
      if (v < nvec) {
        float xf[8], gf[8], wf[8], o[8];
        unpack8(xv[k], xf); unpack8(gv[k], gf); unpack8(wr[v], wf);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (gf[i] * wf[i] - xf[i] * c);
        dr[v] = make_uint4(pack(o[0], o[1]), pack(o[2], o[3]), pack(o[4], o[5]), pack(o[6], o[7]));
      }
    }
  }
  float* prow = partials + size_t(blockIdx.x) * cols;
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k) {
    const int v = threadIdx.x + k * kThreads;
    if (v < nvec) {
#pragma unroll
      for (int i = 0; i < 8; ++i) prow[v * 8 + i] = dw[k][i];
    }
  }
}

__global__ void colsum_noalloc_kernel(const float* __restrict__ partials, float* __restrict__ dw, int parts, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partials[size_t(p) * cols + c];
  dw[c] = s;
}

int fail(char* err, int err_len, int code, const char* msg) {
  if (err != nullptr && err_len > 0) snprintf(err, err_len, "%s", msg);
  return code;
}

}  // namespace

extern "C" int odc_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                                       float* dw, int rows, int cols, void* stream, char* err, int err_len) {
  if (err != nullptr && err_len > 0) err[0] = '\0';
  if (cols <= 0 || cols % 8 != 0) return fail(err, err_len, 1, "cols must be a positive multiple of 8");
  if (cols > ODC_NOALLOC_MAX_COLS) {
    char msg[160];
    snprintf(msg, sizeof(msg), "cols=%d exceeds the built-in workspace (at most %d columns); use the regular entry point",
             cols, ODC_NOALLOC_MAX_COLS);
    return fail(err, err_len, 2, msg);
  }
  if (rows < 0) return fail(err, err_len, 3, "rows must be non-negative");
  if (!dy || !x || !w || !rstd || !dx || !dw) return fail(err, err_len, 4, "null pointer argument");
  // the kernels read and write dy/x/w/dx sixteen bytes at a time and rstd/dw as floats: refuse a
  // pointer that is not aligned for that (a sliced tensor, say) instead of letting the GPU fault
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) |
       reinterpret_cast<uintptr_t>(dx)) & 15)
    return fail(err, err_len, 9, "dy, x, w and dx must be 16-byte aligned");
  if ((reinterpret_cast<uintptr_t>(rstd) | reinterpret_cast<uintptr_t>(dw)) & 3)
    return fail(err, err_len, 10, "rstd and dw must be 4-byte aligned");

  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(err, err_len, 5, cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(err, err_len, 6, "device index out of range");
  float* partials = nullptr;
  {
    // one-time set-up per GPU, with that GPU current: resolve the workspace's DEVICE address
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_partials_addr[dev] == nullptr) {
      void* p = nullptr;
      e = cudaGetSymbolAddress(&p, g_partials);
      if (e != cudaSuccess || p == nullptr) return fail(err, err_len, 7, cudaGetErrorString(e));
      g_partials_addr[dev] = static_cast<float*>(p);
    }
    partials = g_partials_addr[dev];
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int grid = rows < ODC_NOALLOC_MAX_CTAS ? rows : ODC_NOALLOC_MAX_CTAS;
  if (grid > 0) {
    rmsnorm_bwd_noalloc_kernel<<<grid, kThreads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
        static_cast<const __nv_bfloat16*>(w), rstd, static_cast<__nv_bfloat16*>(dx), partials, rows, cols);
  }
  // with rows == 0 there are no partial rows: the sum over zero parts writes dw = 0
  colsum_noalloc_kernel<<<(cols + 255) / 256, 256, 0, s>>>(partials, dw, grid, cols);
  e = cudaGetLastError();
  if (e != cudaSuccess) return fail(err, err_len, 8, cudaGetErrorString(e));
  return 0;
}
