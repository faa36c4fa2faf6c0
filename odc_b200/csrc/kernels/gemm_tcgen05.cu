// bf16 GEMM on the 5th-generation tensor cores (tcgen05) for sm_100a.
//
// Persistent kernel, one CTA per SM, 128 x 256 output tile, K consumed 64 at a time.
//   warp 0      : TMA producer   (one lane; 128-byte-swizzled tiles into a 4-stage smem ring)
//   warp 1      : MMA issuer     (one lane; tcgen05.mma, fp32 accumulators in tensor memory)
//   warps 2..5  : epilogue       (tcgen05.ld -> bias / accumulate / convert -> global stores)
// Two 128x256 fp32 accumulators (all 512 TMEM columns) are used alternately, so the epilogue of
// one tile overlaps the main loop of the next.
//
// Operand layouts (everything row-major in global memory):
//   nt: C[M,N] = A[M,K] * B[N,K]^T   both operands K-major          (forward)
//   nn: C[M,N] = A[M,K] * B[K,N]     B is N-major ("MN-major")      (dgrad)
//   tn: C[M,N] = A[K,M]^T * B[K,N]   both operands MN-major         (wgrad)
// MN-major tiles are fetched as 64-element-wide TMA boxes; the shared-memory descriptors carry
// the matching leading/stride byte offsets, so no transposed copy of an activation is ever made.
// Out-of-range rows/columns are zero-filled by TMA on the way in and masked on the way out.
//
// The reference performs these products with cuBLAS through nn.Linear under autocast
// (examples/llm_training/torch_fsdp2.py:282-283).
#include <cuda.h>
#include <cuda_bf16.h>

#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>

#include "api.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"

namespace odc {

using namespace sm100;

namespace {

constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr int kATile = BM * BK * 2;           // 16 KiB
constexpr int kBTile = BN * BK * 2;           // 32 KiB
constexpr int kStageBytes = kATile + kBTile;  // 48 KiB
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
constexpr uint32_t kTmemCols = 512;
constexpr uint64_t kWaitBudgetNs = 4000000000ull;

struct Params {
  void* c;
  const __nv_bfloat16* bias;
  int M, N, K;
  long long ldc;
  int c_is_f32;
  int accumulate;
  int a_mn, b_mn;  // operand is MN-major
  int tiles_m, tiles_n;
  int* status;
};

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  // barrier block lives after the stage ring
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  const uint32_t full0 = smem_u32(bars);                    // [kStages]
  const uint32_t empty0 = full0 + 8 * kStages;              // [kStages]
  const uint32_t tfull0 = empty0 + 8 * kStages;             // [2]
  const uint32_t tempty0 = tfull0 + 16;                     // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const WaitCtx wc{abort_flag, p.status, kWaitBudgetNs};

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8 * a, 1);
      mbar_init(tempty0 + 8 * a, 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_blocks = (p.K + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      prefetch_tmap(&tmap_a);
      prefetch_tmap(&tmap_b);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % p.tiles_m) * BM;
        const int n0 = (tile / p.tiles_m) * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!(ok = mbar_wait(empty0 + 8 * s, ph ^ 1, wc, 1))) break;
          const uint32_t sa = base + s * kStageBytes;
          const uint32_t sb = sa + kATile;
          const uint32_t bar = full0 + 8 * s;
          mbar_arrive_expect_tx(bar, kStageBytes);
          const int k0 = kb * BK;
          if (!p.a_mn) {
            tma_load_2d(sa, &tmap_a, bar, k0, m0);                 // box {64 k, 128 rows}
          } else {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d(sa + i * 8192, &tmap_a, bar, m0 + 64 * i, k0);
          }
          if (!p.b_mn) {
            tma_load_2d(sb, &tmap_b, bar, k0, n0);                 // box {64 k, 256 rows}
          } else {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sb + i * 8192, &tmap_b, bar, n0 + 64 * i, k0);
          }
        }
      }
      if (!ok) {
        // aborting: give copies already in flight a bounded chance to land before smem is released
        for (int s = 0; s < kStages; ++s) {
          for (int spin = 0; spin < 20000; ++spin)
            if (mbar_try_wait(full0 + 8 * s, 0) || mbar_try_wait(full0 + 8 * s, 1)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, p.a_mn != 0, p.b_mn != 0);
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
      const uint32_t a_kstep = p.a_mn ? 2048u : 32u, b_kstep = p.b_mn ? 2048u : 32u;  // bytes per K=16
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!(ok = mbar_wait(tempty0 + 8 * acc, acc_ph ^ 1, wc, 2))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!(ok = mbar_wait(full0 + 8 * s, ph, wc, 3))) break;
          tc_fence_after();
          const uint32_t sa = base + s * kStageBytes;
          const uint32_t sb = sa + kATile;
#pragma unroll
          for (int j = 0; j < BK / 16; ++j) {
            const uint64_t da = make_smem_desc(sa + j * a_kstep, a_lbo, 1024);
            const uint64_t db = make_smem_desc(sb + j * b_kstep, b_lbo, 1024);
            umma_f16(d_tmem, da, db, idesc, (kb > 0 || j > 0) ? 1u : 0u);
          }
          umma_commit(empty0 + 8 * s);  // stage reusable once these MMAs have read it
        }
        if (ok) umma_commit(tfull0 + 8 * acc);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) belong to this warp
    uint32_t local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
      const int m0 = (tile % p.tiles_m) * BM;
      const int n0 = (tile / p.tiles_m) * BN;
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      if (!(ok = mbar_wait(tfull0 + 8 * acc, acc_ph, wc, 4))) break;
      tc_fence_after();
      const int row = m0 + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(t_row + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) continue;
        float f[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) f[i] = __uint_as_float(r[i]);
        if (p.bias != nullptr) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (col0 + i < p.N) f[i] += __bfloat162float(p.bias[col0 + i]);
        }
        if (row_ok) {
          if (p.c_is_f32) {
            float* crow = static_cast<float*>(p.c) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              if (col0 + v * 4 < p.N) {
                float4 o = make_float4(f[4 * v], f[4 * v + 1], f[4 * v + 2], f[4 * v + 3]);
                if (p.accumulate) {
                  const float4 old = *reinterpret_cast<const float4*>(crow + 4 * v);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(crow + 4 * v) = o;
              }
            }
          } else {
            __nv_bfloat16* crow = static_cast<__nv_bfloat16*>(p.c) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col0 + v * 8 < p.N) {
                if (p.accumulate) {
                  const uint4 old = *reinterpret_cast<const uint4*>(crow + 8 * v);
                  const uint32_t o[4] = {old.x, old.y, old.z, old.w};
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    f[8 * v + 2 * i] += __uint_as_float(o[i] << 16);
                    f[8 * v + 2 * i + 1] += __uint_as_float(o[i] & 0xffff0000u);
                  }
                }
                uint4 o;
                o.x = pack2(f[8 * v], f[8 * v + 1]);
                o.y = pack2(f[8 * v + 2], f[8 * v + 3]);
                o.z = pack2(f[8 * v + 4], f[8 * v + 5]);
                o.w = pack2(f[8 * v + 6], f[8 * v + 7]);
                *reinterpret_cast<uint4*>(crow + 8 * v) = o;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
cudaError_t gemm_bf16(const void* a, const void* b, void* c, int c_kind, const void* bias, int M, int N, int K,
                      int layout, bool accumulate, long long lda, long long ldb, long long ldc, int* status,
                      int sm_count, cudaStream_t stream) {
  if (M == 0 || N == 0) return cudaSuccess;
  if (K == 0) return cudaErrorInvalidValue;
  const bool a_mn = (layout == 2);
  const bool b_mn = (layout != 0);
  // 16-byte rules of TMA: base addresses, row pitches; and of the vector epilogue: N, ldc
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15)
    return cudaErrorMisalignedAddress;
  if ((lda % 8) || (ldb % 8) || (N % 8) || (ldc % (c_kind == kF32 ? 4 : 8))) return cudaErrorInvalidValue;

  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  });
  if (attr_err != cudaSuccess) return attr_err;

  CUtensorMap ta, tb;
  // A: K-major -> dims {K, M}, box {64, 128};  MN-major -> global [K rows, M cols], box {64 (M), 64 (K)}
  if (!a_mn) {
    if (!encode_tile_map_2d(&ta, a, /*inner*/ K, /*outer*/ M, lda * 2, 64, BM)) return cudaErrorInvalidValue;
  } else {
    if (!encode_tile_map_2d(&ta, a, /*inner*/ M, /*outer*/ K, lda * 2, 64, 64)) return cudaErrorInvalidValue;
  }
  if (!b_mn) {
    if (!encode_tile_map_2d(&tb, b, K, N, ldb * 2, 64, BN)) return cudaErrorInvalidValue;
  } else {
    if (!encode_tile_map_2d(&tb, b, N, K, ldb * 2, 64, 64)) return cudaErrorInvalidValue;
  }
  Params p;
  p.c = c;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc;
  p.c_is_f32 = (c_kind == kF32);
  p.accumulate = accumulate ? 1 : 0;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.status = status;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count ? tiles : sm_count;
  gemm_bf16_kernel<<<grid, kThreads, kSmemBytes, stream>>>(ta, tb, p);
  return cudaGetLastError();
}

}  // namespace odc
