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

#include <stdlib.h>

#include <mutex>
#include <stdexcept>
#include <string>
#include <unordered_map>

#include "api.h"
#include "gemm_tcgen05_kernel.cuh"
#include "sm100_ptx.cuh"
#include "tensor_map.h"

namespace odc {

using namespace gemm_impl;

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
cudaError_t gemm_bf16(const void* a, const void* b, void* c, int c_kind, const void* bias, int M, int N, int K,
                      int layout, bool accumulate, long long lda, long long ldb, long long ldc, int* status,
                      int sm_count, cudaStream_t stream, const void* residual, long long ldr, int pair_mode) {
  if (M == 0 || N == 0) return cudaSuccess;
  if (K == 0) return cudaErrorInvalidSymbol;
  static const bool use_pairs = [] {
    const char* e = getenv("ODC_GEMM_PAIR");
    return e == nullptr || e[0] != '0';
  }();
  if (pair_mode == 1 || (pair_mode < 0 && use_pairs)) {
    const cudaError_t e = gemm_bf16_pair(a, b, c, c_kind, bias, M, N, K, layout, accumulate, lda, ldb, ldc, status,
                                         sm_count, stream, residual, ldr);
    if (e != cudaErrorNotSupported || pair_mode == 1) return e;
  }
  const bool a_mn = (layout == 2);
  const bool b_mn = (layout != 0);
  // 16-byte rules of TMA: base addresses, row pitches; and of the vector epilogue: N, ldc
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15)
    return cudaErrorMisalignedAddress;
  if ((lda % 8) || (ldb % 8) || (N % 8) || (ldc % (c_kind == kF32 ? 4 : 8))) return cudaErrorInvalidDevicePointer;

  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<kModePlain>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  });
  if (attr_err != cudaSuccess) return attr_err;

  CUtensorMap ta, tb;
  // A: K-major -> dims {K, M}, box {64, 128};  MN-major -> global [K rows, M cols], box {64 (M), 64 (K)}
  if (!a_mn) {
    if (!encode_tile_map_2d(&ta, a, /*inner*/ K, /*outer*/ M, lda * 2, 64, BM)) return cudaErrorInvalidPitchValue;
  } else {
    if (!encode_tile_map_2d(&ta, a, /*inner*/ M, /*outer*/ K, lda * 2, 64, 64)) return cudaErrorInvalidPitchValue;
  }
  if (!b_mn) {
    if (!encode_tile_map_2d(&tb, b, K, N, ldb * 2, 64, BN)) return cudaErrorInvalidTexture;
  } else {
    if (!encode_tile_map_2d(&tb, b, N, K, ldb * 2, 64, 64)) return cudaErrorInvalidTexture;
  }
  CUtensorMap tc;
  if (c_kind == kF32) {
    if (!encode_tile_map_2d_f32(&tc, c, N, M, ldc * 4, 32, BM)) return cudaErrorInvalidValue;
  } else {
    if (accumulate) return cudaErrorNotSupported;  // accumulation is offered for fp32 outputs
    if (!encode_tile_map_2d(&tc, c, N, M, ldc * 2, 64, BM)) return cudaErrorInvalidValue;
  }
  Params p{};
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
  if (residual != nullptr) {
    if (c_kind != kBF16 || (ldr % 8) || (reinterpret_cast<uintptr_t>(residual) & 15)) return cudaErrorInvalidValue;
    p.residual = static_cast<const __nv_bfloat16*>(residual);
    p.ldr = ldr;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count ? tiles : sm_count;
  gemm_bf16_kernel<kModePlain><<<grid, Roles<kModePlain>::kThreadsTotal, kSmemBytes, stream>>>(ta, tb, tc, OwnerMaps{}, p);
  return cudaGetLastError();
}

}  // namespace odc
