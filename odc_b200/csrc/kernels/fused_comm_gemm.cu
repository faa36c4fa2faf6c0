// Compute + communication in one launch (the two hot paths of on-demand FSDP).
//
// gemm_wgrad_scatter: dW = dY^T X on tcgen05 whose epilogue reduces every output tile straight
//   into the fp32 accumulator of the rank that owns those rows (16-byte red.add over the peer
//   mapping) and finishes with one arrival per owner.  The reference stages the full gradient,
//   copies slices into per-peer mailboxes and has a watcher process add them
//   (odc/fsdp/fsdp2.py:676-710, odc/primitives/scatter_accumulate.py:649-691).
//
// gemm_gather_nt: Y = X W^T where W is row-sharded across ranks.  Two warps per CTA pull the
//   owners' bf16 shards into a local buffer, 256-row panel by panel, while the tensor cores
//   multiply the panels that have already landed; a per-panel counter orders the two.  Every byte
//   of W crosses NVLink once; TMA reads local memory only.  The reference gathers the whole unit
//   with per-peer copies before the first GEMM can start (odc/primitives/gather.py:121-127).
#include <cuda.h>
#include <cuda_bf16.h>

#include <stdlib.h>

#include <mutex>

#include "api.h"
#include "gemm_tcgen05_kernel.cuh"
#include "tensor_map.h"

namespace odc {

using namespace gemm_impl;

// ODC_GEMM_PAIR=0 keeps every GEMM on the single-CTA kernel (for A/B runs); by default shapes of at least one
// 256 x 256 tile run on CTA pairs.
static bool pairs_enabled() {
  static const bool on = [] {
    const char* e = getenv("ODC_GEMM_PAIR");
    return e == nullptr || e[0] != '0';
  }();
  return on;
}

cudaError_t gemm_wgrad_scatter(const void* dy, const void* x, int tokens, int n_out, int k_in, long long ld_dy,
                               long long ld_x, const long long* acc_ptrs, const long long* ctr_ptrs,
                               long long acc_offset, int rows_per_rank, int nranks, float scale,
                               unsigned int* done_slot, int* status, int sm_count, cudaStream_t stream) {
  if (n_out == 0 || k_in == 0 || nranks == 0) return cudaSuccess;
  if (tokens == 0) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x)) & 15) return cudaErrorMisalignedAddress;
  if ((ld_dy % 8) || (ld_x % 8) || (k_in % 8) || (acc_offset % 4)) return cudaErrorInvalidValue;
  if (static_cast<long long>(rows_per_rank) * nranks < n_out) return cudaErrorInvalidValue;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<kModeScatter>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSmemBytes);
  });
  if (attr_err != cudaSuccess) return attr_err;
  CUtensorMap ta, tb;
  // "tn": A = dY viewed as [K = tokens rows, M = n_out cols], B = X as [K = tokens rows, N = k_in cols]
  if (!encode_tile_map_2d(&ta, dy, n_out, tokens, ld_dy * 2, 64, 64)) return cudaErrorInvalidValue;
  if (!encode_tile_map_2d(&tb, x, k_in, tokens, ld_x * 2, 64, 64)) return cudaErrorInvalidValue;
  Params p{};
  p.M = n_out; p.N = k_in; p.K = tokens;
  p.ldc = k_in;
  p.c_is_f32 = 1;
  p.a_mn = 1; p.b_mn = 1;
  p.tiles_m = (n_out + BM - 1) / BM;
  p.tiles_n = (k_in + BN - 1) / BN;
  p.status = status;
  p.acc_ptrs = acc_ptrs; p.ctr_ptrs = ctr_ptrs; p.acc_offset = acc_offset;
  p.rows_per_rank = rows_per_rank; p.nranks = nranks; p.scale = scale; p.done_slot = done_slot;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count ? tiles : sm_count;
  gemm_bf16_kernel<kModeScatter><<<grid, Roles<kModeScatter>::kThreadsTotal, kSmemBytes, stream>>>(ta, tb, ta, OwnerMaps{}, p);
  return cudaGetLastError();
}

cudaError_t gemm_wgrad_scatter_tma(const void* dy, const void* x, int tokens, int n_out, int k_in, long long ld_dy,
                                   long long ld_x, const long long* acc_addrs_host, const long long* ctr_ptrs,
                                   long long acc_offset, int rows_per_rank, int nranks, float scale,
                                   unsigned int* done_slot, int* status, int sm_count, cudaStream_t stream,
                                   int start_rank) {
  if (n_out == 0 || k_in == 0 || nranks == 0) return cudaSuccess;
  if (tokens == 0) return cudaErrorInvalidValue;
  if (pairs_enabled()) {  // CTA pairs (256 x 256 tiles) when the shape allows it
    const cudaError_t e = gemm_wgrad_scatter_pair(dy, x, tokens, n_out, k_in, ld_dy, ld_x, acc_addrs_host, ctr_ptrs,
                                                  acc_offset, rows_per_rank, nranks, scale, done_slot, status, sm_count,
                                                  stream, start_rank);
    if (e != cudaErrorNotSupported) return e;
  }
  if (nranks > kMaxOwners || (rows_per_rank % BM) != 0) return cudaErrorNotSupported;  // caller falls back to red.add
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x)) & 15) return cudaErrorMisalignedAddress;
  if ((ld_dy % 8) || (ld_x % 8) || (k_in % 8) || (acc_offset % 4)) return cudaErrorInvalidValue;
  if (static_cast<long long>(rows_per_rank) * nranks < n_out) return cudaErrorInvalidValue;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<kModeScatterTma>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSmemBytes);
  });
  if (attr_err != cudaSuccess) return attr_err;
  CUtensorMap ta, tb;
  if (!encode_tile_map_2d(&ta, dy, n_out, tokens, ld_dy * 2, 64, 64)) return cudaErrorInvalidValue;
  if (!encode_tile_map_2d(&tb, x, k_in, tokens, ld_x * 2, 64, 64)) return cudaErrorInvalidValue;
  OwnerMaps owners{};
  for (int r = 0; r < nranks; ++r) {
    float* base = reinterpret_cast<float*>(static_cast<uintptr_t>(acc_addrs_host[r])) + acc_offset;
    if (!encode_tile_map_2d_f32(&owners.m[r], base, k_in, rows_per_rank, static_cast<uint64_t>(k_in) * 4, 32, BM))
      return cudaErrorInvalidValue;
  }
  Params p{};
  p.M = n_out; p.N = k_in; p.K = tokens;
  p.ldc = k_in;
  p.c_is_f32 = 1;
  p.a_mn = 1; p.b_mn = 1;
  p.tiles_m = (n_out + BM - 1) / BM;
  p.tiles_n = (k_in + BN - 1) / BN;
  p.status = status;
  p.ctr_ptrs = ctr_ptrs;
  p.rows_per_rank = rows_per_rank; p.nranks = nranks; p.scale = scale; p.done_slot = done_slot;
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count ? tiles : sm_count;
  gemm_bf16_kernel<kModeScatterTma><<<grid, Roles<kModeScatterTma>::kThreadsTotal, kSmemBytes, stream>>>(
      ta, tb, ta, owners, p);
  return cudaGetLastError();
}

cudaError_t gemm_gather_nt(const void* x, const long long* shard_ptrs, void* w_local, void* y, const void* bias,
                           int M, int N, int K, long long ldx, long long ldy, int rows_per_rank, int nranks,
                           int start_rank, unsigned int* panel_flags, int* status, int sm_count,
                           cudaStream_t stream, const void* residual, long long ldr) {
  if (M == 0 || N == 0 || nranks == 0) return cudaSuccess;
  if (K == 0) return cudaErrorInvalidValue;
  if (pairs_enabled()) {
    const cudaError_t e = gemm_gather_pair(false, x, shard_ptrs, w_local, y, bias, M, N, K, ldx, ldy, rows_per_rank,
                                           nranks, panel_flags, status, sm_count, stream, residual, ldr, start_rank);
    if (e != cudaErrorNotSupported) return e;
  }
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w_local) | reinterpret_cast<uintptr_t>(y)) & 15)
    return cudaErrorMisalignedAddress;
  if ((ldx % 8) || (ldy % 8) || (N % 8) || (K % 128)) return cudaErrorInvalidValue;
  if (static_cast<long long>(rows_per_rank) * nranks < N) return cudaErrorInvalidValue;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<kModeGather>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSmemBytes);
  });
  if (attr_err != cudaSuccess) return attr_err;
  CUtensorMap ta, tb;
  if (!encode_tile_map_2d(&ta, x, K, M, ldx * 2, 64, BM)) return cudaErrorInvalidValue;
  if (!encode_tile_map_2d(&tb, w_local, K, N, static_cast<uint64_t>(K) * 2, 64, BN)) return cudaErrorInvalidValue;
  CUtensorMap tc;
  if (!encode_tile_map_2d(&tc, y, N, M, ldy * 2, 64, BM)) return cudaErrorInvalidValue;
  Params p{};
  p.c = y;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldy;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.status = status;
  p.shard_ptrs = shard_ptrs;
  p.b_local = static_cast<unsigned char*>(w_local);
  p.panel_flags = panel_flags;
  p.rows_per_rank = rows_per_rank; p.nranks = nranks; p.start_rank = start_rank;
  p.w_rows = N; p.w_cols = K;
  if (residual != nullptr) {
    if ((ldr % 8) || (reinterpret_cast<uintptr_t>(residual) & 15)) return cudaErrorInvalidValue;
    p.residual = static_cast<const __nv_bfloat16*>(residual);
    p.ldr = ldr;
  }
  cudaError_t e = cudaMemsetAsync(panel_flags, 0, sizeof(unsigned int) * p.tiles_n, stream);
  if (e != cudaSuccess) return e;
  // every CTA also fetches, so use the whole machine even when there are few tiles
  const int grid = sm_count;
  gemm_bf16_kernel<kModeGather><<<grid, Roles<kModeGather>::kThreadsTotal, kSmemBytes, stream>>>(ta, tb, tc, OwnerMaps{}, p);
  return cudaGetLastError();
}

cudaError_t gemm_gather_nn(const void* dy, const long long* shard_ptrs, void* w_local, void* dx, int M, int n_out,
                           int k_in, long long lddy, long long lddx, int rows_per_rank, int nranks,
                           unsigned int* group_flags, int* status, int sm_count, cudaStream_t stream,
                           int start_rank) {
  // dx[M, k_in] = dy[M, n_out] * W[n_out, k_in]; W's rows (the reduction dimension) are gathered
  if (M == 0 || k_in == 0 || nranks == 0) return cudaSuccess;
  if (n_out == 0) return cudaErrorInvalidValue;
  if (pairs_enabled()) {
    const cudaError_t e = gemm_gather_pair(true, dy, shard_ptrs, w_local, dx, nullptr, M, n_out, k_in, lddy, lddx,
                                           rows_per_rank, nranks, group_flags, status, sm_count, stream, nullptr, 0,
                                           start_rank);
    if (e != cudaErrorNotSupported) return e;
  }
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(w_local) | reinterpret_cast<uintptr_t>(dx)) & 15)
    return cudaErrorMisalignedAddress;
  if ((lddy % 8) || (lddx % 8) || (n_out % 8) || (k_in % 128)) return cudaErrorInvalidValue;
  if (static_cast<long long>(rows_per_rank) * nranks < n_out) return cudaErrorInvalidValue;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_bf16_kernel<kModeGather>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSmemBytes);
  });
  if (attr_err != cudaSuccess) return attr_err;
  CUtensorMap ta, tb, tc;
  if (!encode_tile_map_2d(&ta, dy, n_out, M, lddy * 2, 64, BM)) return cudaErrorInvalidValue;
  // B is MN-major: rows = reduction index, box {64 output columns, 64 reduction rows}
  if (!encode_tile_map_2d(&tb, w_local, k_in, n_out, static_cast<uint64_t>(k_in) * 2, 64, 64)) return cudaErrorInvalidValue;
  if (!encode_tile_map_2d(&tc, dx, k_in, M, lddx * 2, 64, BM)) return cudaErrorInvalidValue;
  Params p{};
  p.c = dx;
  p.M = M; p.N = k_in; p.K = n_out;
  p.ldc = lddx;
  p.b_mn = 1;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (k_in + BN - 1) / BN;
  p.status = status;
  p.shard_ptrs = shard_ptrs;
  p.b_local = static_cast<unsigned char*>(w_local);
  p.panel_flags = group_flags;
  p.rows_per_rank = rows_per_rank; p.nranks = nranks;
  p.w_rows = n_out; p.w_cols = k_in;
  cudaError_t e = cudaMemsetAsync(group_flags, 0, sizeof(unsigned int) * ((n_out + BN - 1) / BN), stream);
  if (e != cudaSuccess) return e;
  const int grid = sm_count;
  gemm_bf16_kernel<kModeGather><<<grid, Roles<kModeGather>::kThreadsTotal, kSmemBytes, stream>>>(ta, tb, tc, OwnerMaps{}, p);
  return cudaGetLastError();
}

}  // namespace odc
