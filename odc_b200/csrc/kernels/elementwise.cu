// Memory-bound ops of the decoder, each a single pass with 16-byte accesses and fp32 math:
// RMSNorm fwd/bwd, rotary embedding on a fused qkv activation, SwiGLU fwd/bwd, softmax
// cross-entropy that turns logits into their gradient in place, AdamW on flat shards (also
// refreshing the low-precision copy that peers gather), casts and a sum-of-squares reduction.
// The reference runs these as eager PyTorch ops inside Hugging Face modules
// (examples/llm_training/torch_fsdp2.py:164, lm_head.py:7-59) and torch.optim.AdamW (:322).
#include <cuda_bf16.h>

#include "api.h"

namespace odc {
namespace {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  f[0] = lo(u.x); f[1] = hi(u.x); f[2] = lo(u.y); f[3] = hi(u.y);
  f[4] = lo(u.z); f[5] = hi(u.z); f[6] = lo(u.w); f[7] = hi(u.w);
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  return make_uint4(pack(f[0], f[1]), pack(f[2], f[3]), pack(f[4], f[5]), pack(f[6], f[7]));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// block-wide sum, result in every thread; `red` holds 32 floats
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : 0.f;
  return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nw) ? red[lane] : -INFINITY;
  return warp_max(t);
}

// ------------------------------------------------------------------------- RMSNorm ----------
// A row is handled by R warps (R = 1 up to 2048 columns, 2 up to 4096, 4 up to 8192); a lane keeps up to 8
// 16-byte pieces of the row in registers with all loads in flight at once.  With R = 1 the row statistics
// need only warp shuffles and no block-wide barrier sits on the critical path.
constexpr int kNormThreads = 256;
constexpr int kNormWarps = kNormThreads / 32;
constexpr int kNormVec = 8;

// sum over the R warps that share a row (R > 1 only); every thread of the CTA must call it
template <int R>
__device__ __forceinline__ float row_sum(float v, float* red, int warp, int lane) {
  v = warp_sum(v);
  if constexpr (R == 1) return v;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int first = warp - warp % R;
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < R; ++i) t += red[first + i];
  return t;
}

template <int R>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, bf16* __restrict__ y,
                   float* __restrict__ rstd_out, int rows, int cols, float eps) {
  __shared__ float red[kNormWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = warp % R;                       // which part of the row this warp covers
  constexpr int kRowsPerIter = kNormWarps / R;
  const int nvec = cols / 8;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const int iters = (rows + gridDim.x * kRowsPerIter - 1) / (gridDim.x * kRowsPerIter);
  for (int it = 0; it < iters; ++it) {
    const int row = (it * gridDim.x + blockIdx.x) * kRowsPerIter + warp / R;
    const bool live = row < rows;
    const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(live ? row : 0) * cols);
    uint4 xv[kNormVec];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < kNormVec; ++k) {
      const int v = (sub * kNormVec + k) * 32 + lane;
      if (live && v < nvec) xv[k] = xr[v];
    }
#pragma unroll
    for (int k = 0; k < kNormVec; ++k) {
      const int v = (sub * kNormVec + k) * 32 + lane;
      if (live && v < nvec) {
        float f[8];
        unpack8(xv[k], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
      }
    }
    ss = row_sum<R>(ss, red, warp, lane);
    if (!live) continue;
    const float rstd = rsqrtf(ss / cols + eps);
    if (lane == 0 && sub == 0) rstd_out[row] = rstd;
    uint4* yr = reinterpret_cast<uint4*>(y + size_t(row) * cols);
#pragma unroll
    for (int k = 0; k < kNormVec; ++k) {
      const int v = (sub * kNormVec + k) * 32 + lane;
      if (v < nvec) {
        float f[8], g[8];
        unpack8(xv[k], f);
        unpack8(wr[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * g[i];
        yr[v] = pack8(f);
      }
    }
  }
}

// dx = rstd * (dy*w - x * rstd^2 * mean(dy*w*x)).  A row is handled by R warps and a lane keeps V 16-byte pieces of
// x and dy in registers (V <= 4, so the kernel fits two CTAs per SM and both keep loads in flight); each lane
// accumulates dw for its own columns over all rows it handles, the warps of a CTA combine through shared memory,
// and the CTA then either adds its sums into dw (kAtomic: dw zeroed before the launch, one launch in total) or
// writes one row of partial sums for a second, fixed-order pass.
template <int R, int V, bool kAtomic>
__global__ void __launch_bounds__(kNormThreads, 2)
rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                   const float* __restrict__ rstd_in, bf16* __restrict__ dx, float* __restrict__ partial,
                   float* __restrict__ dw_out, int rows, int cols, const bf16* __restrict__ dres) {
  extern __shared__ float dw_smem[];  // [cols]
  __shared__ float red[kNormWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = warp % R;
  constexpr int kRowsPerIter = kNormWarps / R;
  const int nvec = cols / 8;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) dw_smem[c] = 0.f;
  float dw[V][8];
#pragma unroll
  for (int k = 0; k < V; ++k)
#pragma unroll
    for (int i = 0; i < 8; ++i) dw[k][i] = 0.f;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const int iters = (rows + gridDim.x * kRowsPerIter - 1) / (gridDim.x * kRowsPerIter);
  for (int it = 0; it < iters; ++it) {
    const int row = (it * gridDim.x + blockIdx.x) * kRowsPerIter + warp / R;
    const bool live = row < rows;
    const uint4* xr = reinterpret_cast<const uint4*>(x + size_t(live ? row : 0) * cols);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + size_t(live ? row : 0) * cols);
    const float rstd = live ? rstd_in[row] : 0.f;
    uint4 xv[V], gv[V];
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int v = (sub * V + k) * 32 + lane;
      if (live && v < nvec) {
        xv[k] = xr[v];
        gv[k] = gr[v];
      }
    }
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int v = (sub * V + k) * 32 + lane;
      if (live && v < nvec) {
        float xf[8], gf[8], wf[8];
        unpack8(xv[k], xf);
        unpack8(gv[k], gf);
        unpack8(wr[v], wf);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          dot += gf[i] * wf[i] * xf[i];
          dw[k][i] += gf[i] * xf[i] * rstd;
        }
      }
    }
    dot = row_sum<R>(dot, red, warp, lane);
    if (!live) continue;
    const float c = dot * rstd * rstd / cols;
    uint4* dr = reinterpret_cast<uint4*>(dx + size_t(row) * cols);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      const int v = (sub * V + k) * 32 + lane;
      if (v < nvec) {
        float xf[8], gf[8], wf[8], o[8];
        unpack8(xv[k], xf);
        unpack8(gv[k], gf);
        unpack8(wr[v], wf);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = rstd * (gf[i] * wf[i] - xf[i] * c);
        if (dres != nullptr) {  // gradient that reached x through the residual path: one pass instead of a separate add
          float rf[8];
          unpack8(reinterpret_cast<const uint4*>(dres + size_t(row) * cols)[v], rf);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] += rf[i];
        }
        dr[v] = pack8(o);
      }
    }
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int v = (sub * V + k) * 32 + lane;
    if (v < nvec) {
#pragma unroll
      for (int i = 0; i < 8; ++i) atomicAdd(&dw_smem[v * 8 + i], dw[k][i]);
    }
  }
  __syncthreads();
  if constexpr (kAtomic) {
    for (int c = threadIdx.x; c < cols; c += blockDim.x) atomicAdd(dw_out + c, dw_smem[c]);
  } else {
    float* prow = partial + size_t(blockIdx.x) * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) prow[c] = dw_smem[c];
  }
}

__global__ void colsum_kernel(const float* __restrict__ partial, float* __restrict__ out, int parts, int cols) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  for (int p = 0; p < parts; ++p) s += partial[size_t(p) * cols + c];
  out[c] = s;
}

// ------------------------------------------------------------------------- RoPE -------------
// one CTA per token; cos/sin of the head_dim/2 angles computed once and reused by all heads
__global__ void __launch_bounds__(128)
rope_qkv_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, const long long* __restrict__ pos, int n_q,
                int n_kv, int head_dim, float log2_theta, float sign) {
  extern __shared__ float cs[];  // [head_dim/2] cos, [head_dim/2] sin
  const int t = blockIdx.x;
  const int half = head_dim / 2;
  const float p = static_cast<float>(pos[t]);
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float inv = exp2f(-log2_theta * (2.0f * i) / head_dim);
    float s, c;
    sincosf(p * inv, &s, &c);
    cs[i] = c;
    cs[half + i] = s * sign;
  }
  __syncthreads();
  const int width = (n_q + 2 * n_kv) * head_dim;
  const bf16* row = in + size_t(t) * width;
  bf16* orow = out + size_t(t) * width;
  const int rot_heads = n_q + n_kv;
  const int vec_per_half = half / 8;
  const int rot_items = rot_heads * vec_per_half;
  for (int it = threadIdx.x; it < rot_items; it += blockDim.x) {
    const int h = it / vec_per_half, j = (it % vec_per_half) * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(row + h * head_dim + j);
    const uint4 b = *reinterpret_cast<const uint4*>(row + h * head_dim + half + j);
    float x1[8], x2[8], o1[8], o2[8];
    unpack8(a, x1);
    unpack8(b, x2);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float c = cs[j + i], s = cs[half + j + i];
      o1[i] = x1[i] * c - x2[i] * s;
      o2[i] = x2[i] * c + x1[i] * s;
    }
    *reinterpret_cast<uint4*>(orow + h * head_dim + j) = pack8(o1);
    *reinterpret_cast<uint4*>(orow + h * head_dim + half + j) = pack8(o2);
  }
  const int v_off = rot_heads * head_dim;
  const int v_vecs = n_kv * head_dim / 8;
  for (int it = threadIdx.x; it < v_vecs; it += blockDim.x)
    *reinterpret_cast<uint4*>(orow + v_off + it * 8) = *reinterpret_cast<const uint4*>(row + v_off + it * 8);
}

// ------------------------------------------------------------------------- SwiGLU -----------
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, long long rows, int f) {
  const int vec_per_row = f / 8;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + r * 2 * f + c);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + r * 2 * f + f + c);
    float gf[8], uf[8], o[8];
    unpack8(g, gf);
    unpack8(u, uf);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = gf[k] / (1.f + __expf(-gf[k])) * uf[k];
    *reinterpret_cast<uint4*>(out + r * f + c) = pack8(o);
  }
}

__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ gu, bf16* __restrict__ dgu, long long rows,
                  int f) {
  const int vec_per_row = f / 8;
  const long long total = rows * vec_per_row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row;
    const int c = static_cast<int>(i % vec_per_row) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gu + r * 2 * f + c);
    const uint4 u = *reinterpret_cast<const uint4*>(gu + r * 2 * f + f + c);
    const uint4 d = *reinterpret_cast<const uint4*>(dy + r * f + c);
    float gf[8], uf[8], df[8], dg[8], du[8];
    unpack8(g, gf);
    unpack8(u, uf);
    unpack8(d, df);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sig = 1.f / (1.f + __expf(-gf[k]));
      const float silu = gf[k] * sig;
      du[k] = df[k] * silu;
      dg[k] = df[k] * uf[k] * (sig + silu * (1.f - sig));
    }
    *reinterpret_cast<uint4*>(dgu + r * 2 * f + c) = pack8(dg);
    *reinterpret_cast<uint4*>(dgu + r * 2 * f + f + c) = pack8(du);
  }
}

// ------------------------------------------------------------------------- cross-entropy ----
// one CTA per row; pass 1: online max / sum-exp; pass 2: logits <- scale * (softmax - onehot)
// kForwardOnly: pass 1 only, the logits stay as they are and the row's log-probability of its label
// (0 for an ignored row) goes to per_token[row]; the scale and the summed loss are not used.
constexpr int kCeThreads = 1024;
template <bool kForwardOnly>
__global__ void __launch_bounds__(kCeThreads)
ce_fwd_bwd_kernel(bf16* __restrict__ logits, const long long* __restrict__ labels, const float* __restrict__ loss_scale,
                  float* __restrict__ loss, int vocab, long long ignore_index, float* __restrict__ per_token) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  bf16* lr = logits + size_t(row) * vocab;
  const long long label = labels[row];
  const float scale = (!kForwardOnly && loss_scale) ? loss_scale[row] : 1.f;
  const bool ignored = (label == ignore_index) || scale == 0.f;
  const int nvec = vocab / 8;
  uint4* lv = reinterpret_cast<uint4*>(lr);
  if (ignored) {
    if constexpr (kForwardOnly) {
      if (threadIdx.x == 0) per_token[row] = 0.f;
    } else {
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) lv[v] = make_uint4(0, 0, 0, 0);
      for (int j = nvec * 8 + threadIdx.x; j < vocab; j += blockDim.x) lr[j] = __float2bfloat16(0.f);
    }
    return;
  }
  float m = -INFINITY, s = 0.f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(lv[v], f);
    float mx = f[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) mx = fmaxf(mx, f[i]);
    if (mx > m) {
      s *= __expf(m - mx);
      m = mx;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) s += __expf(f[i] - m);
  }
  for (int j = nvec * 8 + threadIdx.x; j < vocab; j += blockDim.x) {
    const float f = __bfloat162float(lr[j]);
    if (f > m) {
      s *= __expf(m - f);
      m = f;
    }
    s += __expf(f - m);
  }
  const float gm = block_max(m, red);
  s = (m == -INFINITY) ? 0.f : s * __expf(m - gm);
  const float gs = block_sum(s, red);
  const float lse = gm + logf(gs);
  if constexpr (kForwardOnly) {
    if (threadIdx.x == 0) per_token[row] = __bfloat162float(lr[label]) - lse;
    return;
  }
  if (threadIdx.x == 0) atomicAdd(loss, scale * (lse - __bfloat162float(lr[label])));
  __syncthreads();  // the label logit is read above before anyone overwrites it
  const float inv = 1.f / gs;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    unpack8(lv[v], f);
    const int base = v * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float p = __expf(f[i] - gm) * inv;
      if (base + i == label) p -= 1.f;
      f[i] = p * scale;
    }
    lv[v] = pack8(f);
  }
  for (int j = nvec * 8 + threadIdx.x; j < vocab; j += blockDim.x) {
    float p = __expf(__bfloat162float(lr[j]) - gm) * inv;
    if (j == label) p -= 1.f;
    lr[j] = __float2bfloat16(p * scale);
  }
}

// ------------------------------------------------------------------------- AdamW ------------
template <typename GT>
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p, const GT* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
             bf16* __restrict__ p_lowp, size_t n, float lr, float beta1, float beta2, float eps, float wd,
             float inv_bc1, float inv_sqrt_bc2, float grad_scale) {
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
    float gi;
    if constexpr (sizeof(GT) == 4) gi = g[i]; else gi = __bfloat162float(g[i]);
    gi *= grad_scale;
    float pi = p[i] * (1.f - lr * wd);
    const float mi = beta1 * m[i] + (1.f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
    const float denom = sqrtf(vi) * inv_sqrt_bc2 + eps;
    pi -= lr * inv_bc1 * mi / denom;
    p[i] = pi;
    m[i] = mi;
    v[i] = vi;
    if (p_lowp) p_lowp[i] = __float2bfloat16(pi);
  }
}

__global__ void __launch_bounds__(256)
cast_f32_bf16_kernel(const float* __restrict__ in, bf16* __restrict__ out, size_t n) {
  const size_t nvec = n / 8;
  for (size_t v = size_t(blockIdx.x) * blockDim.x + threadIdx.x; v < nvec; v += size_t(gridDim.x) * blockDim.x) {
    const float4 a = *reinterpret_cast<const float4*>(in + v * 8);
    const float4 b = *reinterpret_cast<const float4*>(in + v * 8 + 4);
    *reinterpret_cast<uint4*>(out + v * 8) = make_uint4(pack(a.x, a.y), pack(a.z, a.w), pack(b.x, b.y), pack(b.z, b.w));
  }
  if (blockIdx.x == 0)
    for (size_t j = nvec * 8 + threadIdx.x; j < n; j += blockDim.x) out[j] = __float2bfloat16(in[j]);
}

template <typename T>
__global__ void __launch_bounds__(256) sumsq_kernel(const T* __restrict__ x, size_t n, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += size_t(gridDim.x) * blockDim.x) {
    float f;
    if constexpr (sizeof(T) == 4) f = x[i]; else f = __bfloat162float(x[i]);
    s += f * f;
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) atomicAdd(out, s);
}

int cap_grid(long long work_items, int threads, int sm_count, int per_sm) {
  long long g = (work_items + threads - 1) / threads;
  const long long cap = (long long)sm_count * per_sm;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

template <int R>
cudaError_t rmsnorm_fwd_t(const void* x, const void* w, void* y, float* rstd, int rows, int cols, float eps, int sm_count,
                          cudaStream_t stream) {
  const int want = (rows + kNormWarps / R - 1) / (kNormWarps / R);
  const int grid = want < sm_count * 8 ? want : sm_count * 8;
  rmsnorm_fwd_kernel<R><<<grid, kNormThreads, 0, stream>>>(static_cast<const bf16*>(x), static_cast<const bf16*>(w),
                                                           static_cast<bf16*>(y), rstd, rows, cols, eps);
  return cudaGetLastError();
}

template <int R, int V>
cudaError_t rmsnorm_bwd_t(const void* dy, const void* x, const void* w, const float* rstd, void* dx, float* partial,
                          float* dw, int rows, int cols, int grid, cudaStream_t stream, const void* dres) {
  if (partial == nullptr) {
    rmsnorm_bwd_kernel<R, V, true><<<grid, kNormThreads, cols * sizeof(float), stream>>>(
        static_cast<const bf16*>(dy), static_cast<const bf16*>(x), static_cast<const bf16*>(w), rstd,
        static_cast<bf16*>(dx), nullptr, dw, rows, cols, static_cast<const bf16*>(dres));
  } else {
    rmsnorm_bwd_kernel<R, V, false><<<grid, kNormThreads, cols * sizeof(float), stream>>>(
        static_cast<const bf16*>(dy), static_cast<const bf16*>(x), static_cast<const bf16*>(w), rstd,
        static_cast<bf16*>(dx), partial, dw, rows, cols, static_cast<const bf16*>(dres));
  }
  return cudaGetLastError();
}

}  // namespace

cudaError_t launch_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int cols, float eps,
                               int sm_count, cudaStream_t stream) {
  if (cols % 8 != 0 || cols > 8192) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  if (cols <= 2048) return rmsnorm_fwd_t<1>(x, w, y, rstd, rows, cols, eps, sm_count, stream);
  if (cols <= 4096) return rmsnorm_fwd_t<2>(x, w, y, rstd, rows, cols, eps, sm_count, stream);
  return rmsnorm_fwd_t<4>(x, w, y, rstd, rows, cols, eps, sm_count, stream);
}

int rmsnorm_bwd_grid(int rows, int sm_count) {
  const int want = (rows + kNormWarps - 1) / kNormWarps;
  const int g = sm_count * 2;
  return want < g ? (want < 1 ? 1 : want) : g;
}

// partial == nullptr: single launch, the CTAs add their column sums into dw (zeroed here first; the order of the
// additions varies from run to run).  partial = [grid, cols] scratch: per-CTA sums, then a fixed-order column pass.
cudaError_t launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                               float* partial, float* dw, int rows, int cols, int grid, cudaStream_t stream,
                               const void* dres) {
  if (cols % 8 != 0 || cols > 8192) return cudaErrorInvalidValue;
  cudaError_t e;
  if (partial == nullptr) {
    e = cudaMemsetAsync(dw, 0, sizeof(float) * cols, stream);
    if (e != cudaSuccess) return e;
    if (rows == 0) return cudaSuccess;
  }
  if (cols <= 1024) e = rmsnorm_bwd_t<1, 4>(dy, x, w, rstd, dx, partial, dw, rows, cols, grid, stream, dres);
  else if (cols <= 2048) e = rmsnorm_bwd_t<2, 4>(dy, x, w, rstd, dx, partial, dw, rows, cols, grid, stream, dres);
  else if (cols <= 4096) e = rmsnorm_bwd_t<4, 4>(dy, x, w, rstd, dx, partial, dw, rows, cols, grid, stream, dres);
  else e = rmsnorm_bwd_t<8, 4>(dy, x, w, rstd, dx, partial, dw, rows, cols, grid, stream, dres);
  if (e != cudaSuccess) return e;
  if (partial != nullptr) {
    colsum_kernel<<<(cols + 255) / 256, 256, 0, stream>>>(partial, dw, grid, cols);
    e = cudaGetLastError();
  }
  return e;
}

cudaError_t launch_rope_qkv(const void* in, void* out, const long long* pos, int tokens, int n_q, int n_kv,
                            int head_dim, float theta, bool inverse, cudaStream_t stream) {
  if (head_dim % 16 != 0) return cudaErrorInvalidValue;
  if (tokens == 0) return cudaSuccess;
  rope_qkv_kernel<<<tokens, 128, head_dim * sizeof(float), stream>>>(
      static_cast<const bf16*>(in), static_cast<bf16*>(out), pos, n_q, n_kv, head_dim, log2f(theta),
      inverse ? -1.f : 1.f);
  return cudaGetLastError();
}

cudaError_t launch_swiglu_fwd(const void* gate_up, void* out, long long rows, int f, int sm_count,
                              cudaStream_t stream) {
  if (f % 8 != 0) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  swiglu_fwd_kernel<<<cap_grid(rows * (f / 8), 256, sm_count, 16), 256, 0, stream>>>(
      static_cast<const bf16*>(gate_up), static_cast<bf16*>(out), rows, f);
  return cudaGetLastError();
}

cudaError_t launch_swiglu_bwd(const void* dy, const void* gate_up, void* dgate_up, long long rows, int f,
                              int sm_count, cudaStream_t stream) {
  if (f % 8 != 0) return cudaErrorInvalidValue;
  if (rows == 0) return cudaSuccess;
  swiglu_bwd_kernel<<<cap_grid(rows * (f / 8), 256, sm_count, 16), 256, 0, stream>>>(
      static_cast<const bf16*>(dy), static_cast<const bf16*>(gate_up), static_cast<bf16*>(dgate_up), rows, f);
  return cudaGetLastError();
}

cudaError_t launch_ce_fwd_bwd(void* logits, const long long* labels, const float* loss_scale, float* loss,
                              int rows, int vocab, long long ignore_index, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  if (vocab % 8 != 0) return cudaErrorInvalidValue;  // rows must stay 16-byte aligned
  ce_fwd_bwd_kernel<false><<<rows, kCeThreads, 0, stream>>>(static_cast<bf16*>(logits), labels, loss_scale, loss, vocab,
                                                            ignore_index, nullptr);
  return cudaGetLastError();
}

cudaError_t launch_token_logprobs(const void* logits, const long long* labels, float* per_token, int rows, int vocab,
                                  long long ignore_index, cudaStream_t stream) {
  if (rows == 0) return cudaSuccess;
  if (vocab % 8 != 0 || per_token == nullptr) return cudaErrorInvalidValue;
  // the forward-only instantiation never writes through the logits pointer
  ce_fwd_bwd_kernel<true><<<rows, kCeThreads, 0, stream>>>(static_cast<bf16*>(const_cast<void*>(logits)), labels, nullptr,
                                                           nullptr, vocab, ignore_index, per_token);
  return cudaGetLastError();
}

cudaError_t launch_adamw(float* p, const void* g, int g_kind, float* m, float* v, void* p_lowp, size_t n, float lr,
                         float beta1, float beta2, float eps, float wd, float bc1, float bc2, float grad_scale,
                         int sm_count, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  const int grid = cap_grid(static_cast<long long>(n), 256, sm_count, 16);
  const float inv_bc1 = 1.f / bc1, inv_sqrt_bc2 = 1.f / sqrtf(bc2);
  if (g_kind == kF32)
    adamw_kernel<float><<<grid, 256, 0, stream>>>(p, static_cast<const float*>(g), m, v, static_cast<bf16*>(p_lowp),
                                                  n, lr, beta1, beta2, eps, wd, inv_bc1, inv_sqrt_bc2, grad_scale);
  else if (g_kind == kBF16)
    adamw_kernel<bf16><<<grid, 256, 0, stream>>>(p, static_cast<const bf16*>(g), m, v, static_cast<bf16*>(p_lowp), n,
                                                 lr, beta1, beta2, eps, wd, inv_bc1, inv_sqrt_bc2, grad_scale);
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

cudaError_t launch_cast_f32_to_bf16(const float* in, void* out, size_t n, int sm_count, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  cast_f32_bf16_kernel<<<cap_grid(static_cast<long long>(n / 8 + 1), 256, sm_count, 16), 256, 0, stream>>>(
      in, static_cast<bf16*>(out), n);
  return cudaGetLastError();
}

cudaError_t launch_sumsq(const void* x, int kind, size_t n, float* out, int sm_count, cudaStream_t stream) {
  if (n == 0) return cudaSuccess;
  const int grid = cap_grid(static_cast<long long>(n), 256, sm_count, 8);
  if (kind == kF32)
    sumsq_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(x), n, out);
  else
    sumsq_kernel<bf16><<<grid, 256, 0, stream>>>(static_cast<const bf16*>(x), n, out);
  return cudaGetLastError();
}

}  // namespace odc
