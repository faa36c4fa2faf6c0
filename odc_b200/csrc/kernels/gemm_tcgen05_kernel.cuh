// Kernel body shared by the plain GEMM and its two communication-fused variants (see
// gemm_tcgen05.cu for the design of the main loop).
//   kModePlain   : C is written (or accumulated) locally.
//   kModeScatter : weight-gradient GEMM whose epilogue issues 16-byte red.add.f32 straight into the
//                  fp32 accumulator of the rank that owns each output row, then signals arrival.
//   kModeScatterTma : same result, but output boxes are staged in shared memory and added into the owner's
//                  accumulator by the TMA unit (bulk reduce-add through the peer mapping), which keeps the
//                  link busy with far fewer issued instructions than per-thread reductions.
//   kModeGather  : forward GEMM whose B operand (a row-sharded weight) is pulled from the owners'
//                  shards into local memory by two extra warps per CTA while the tensor cores work
//                  on panels that have already landed; TMA only ever reads this GPU's own memory.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>

#include "api.h"
#include "sm100_ptx.cuh"

namespace odc {
namespace gemm_impl {

using namespace sm100;


constexpr int BM = 128, BN = 256, BK = 64;
constexpr int kStages = 4;
constexpr int kThreads = 192;
constexpr int kATile = BM * BK * 2;           // 16 KiB
constexpr int kBTile = BN * BK * 2;           // 32 KiB
constexpr int kStageBytes = kATile + kBTile;  // 48 KiB
constexpr int kStagingBytes = 128 * 128;    // one output box: 128 rows x 128 bytes (64 bf16 or 32 fp32 columns)
constexpr int kSmemBytes = kStages * kStageBytes + 2 * kStagingBytes + 1024 /*align*/ + 256 /*barriers*/;
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
  const __nv_bfloat16* residual;  // optional [M, N] bf16 added to a bf16 output (row pitch ldr)
  long long ldr;
  // --- kModeScatter: the epilogue adds the tile into the owners' fp32 accumulators ---
  const long long* acc_ptrs;   // [nranks] base address of the accumulator on each owner
  const long long* ctr_ptrs;   // [nranks] arrival counters
  long long acc_offset;        // element offset of this parameter inside an accumulator
  int rows_per_rank;           // output rows owned by one rank
  int nranks;
  float scale;
  unsigned int* done_slot;     // self-resetting CTA completion counter (scratch)
  // --- kModeGather: operand B is assembled from the owners' shards while the GEMM runs ---
  const long long* shard_ptrs; // [nranks] base address of each owner's [rows_per_rank, w_cols] bf16 shard
  unsigned char* b_local;      // local [w_rows, w_cols] bf16 buffer the shards are gathered into (tensor map B covers it)
  unsigned int* panel_flags;   // [ceil(w_rows / 256)] chunks landed per 256-row group (zeroed before launch)
  int w_rows, w_cols;          // gathered matrix: [N, K] when B is K-major (y = x W^T), [K, N] when MN-major (dx = dy W)
  int start_rank;
};

constexpr int kModePlain = 0, kModeScatter = 1, kModeGather = 2, kModeScatterTma = 3;
constexpr int kMaxOwners = 8;
// one fp32 tensor map per owner's accumulator region (kModeScatterTma)
struct OwnerMaps {
  CUtensorMap m[kMaxOwners];
};
// warp roles: 0 = TMA, 1 = MMA, then epilogue warps, then (gather mode) shard-fetch warps
template <int kMode> struct Roles {
  static constexpr int kEpilogueWarps = (kMode == kModeScatter) ? 8 : 4;  // remote reductions need more issue slots
  static constexpr int kFetchWarps = (kMode == kModeGather) ? 4 : 0;
  static constexpr int kThreadsTotal = 32 * (2 + kEpilogueWarps + kFetchWarps);
};
constexpr int kFetchWarpBytes = 16384;                  // moved by one fetch warp between two flag updates
constexpr int kFetchChunkBytes = 4 * kFetchWarpBytes;   // per CTA and step

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int kMode>
__global__ void __launch_bounds__(Roles<kMode>::kThreadsTotal, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ OwnerMaps owners, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  // barrier block lives after the stage ring
  uint8_t* staging = smem + kStages * kStageBytes;               // 2 output boxes for the TMA-store epilogue
  const uint32_t staging_u32 = base + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 2 * kStagingBytes);
  const uint32_t full0 = smem_u32(bars);                    // [kStages]
  const uint32_t empty0 = full0 + 8 * kStages;              // [kStages]
  const uint32_t tfull0 = empty0 + 8 * kStages;             // [2]
  const uint32_t tempty0 = tfull0 + 16;                     // [2]
  const uint32_t sready0 = tempty0 + 16;                    // [2] staging box written by all epilogue warps
  const uint32_t sfree0 = sready0 + 16;                     // [2] staging box read by the TMA unit
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 8);
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
      mbar_init(tempty0 + 8 * a, Roles<kMode>::kEpilogueWarps);  // one arrival per epilogue warp
      mbar_init(sready0 + 8 * a, 4);
      mbar_init(sfree0 + 8 * a, 1);
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
      // gather mode: wait (bounded) until every chunk of 256-row group `g` of the gathered matrix is in local memory
      int groups_ready = 0;  // groups [0, groups_ready) are known to be complete
      auto wait_group = [&](int g) -> bool {
        if (g < groups_ready) return true;
        const long long group_bytes = static_cast<long long>(min(BN, p.w_rows - g * BN)) * p.w_cols * 2;
        const unsigned int target = static_cast<unsigned int>((group_bytes + kFetchChunkBytes - 1) / kFetchChunkBytes) * 4u;
        const uint64_t t0 = globaltimer_ns();
        unsigned int seen;
        while (true) {
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.panel_flags + g) : "memory");
          if (seen >= target) break;
          if (*abort_flag) return false;
          if (globaltimer_ns() - t0 > kWaitBudgetNs) {
            *abort_flag = 1;
            report(p.status, kErrPipelineTimeout, 5, g);
            return false;
          }
          __nanosleep(64);
        }
        asm volatile("fence.proxy.async;" ::: "memory");  // generic-proxy stores -> visible to TMA reads
        // the reduction dimension is walked in order, so in the MN-major case all earlier groups are complete too
        if (p.b_mn) groups_ready = g + 1;
        return true;
      };
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % p.tiles_m) * BM;
        const int n0 = (tile / p.tiles_m) * BN;
        if constexpr (kMode == kModeGather) {
          // B K-major (forward): the 256 weight rows this tile multiplies must have landed in local memory first
          if (!p.b_mn && !(ok = wait_group(tile / p.tiles_m))) break;
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if constexpr (kMode == kModeGather) {
            // B MN-major (input gradient): the gathered rows are the reduction dimension, 4 k-blocks per group
            if (p.b_mn && !(ok = wait_group((kb * BK) / BN))) break;
          }
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
  } else if (kMode == kModeGather && warp >= 2 + Roles<kMode>::kEpilogueWarps) {
    // ------------------------------------------------------------------ shard fetch
    // Copy the owners' shards into the local B buffer in address order (= panel order): 64 KiB per
    // step and CTA, 16 KiB per warp with 16 x 16-byte loads in flight per lane; after its part a warp
    // makes the stores visible and counts them on the panel's flag.
    const int fw = warp - (2 + Roles<kMode>::kEpilogueWarps);
    const long long total_bytes = static_cast<long long>(p.w_rows) * p.w_cols * 2;
    const long long shard_bytes = static_cast<long long>(p.rows_per_rank) * p.w_cols * 2;
    const long long panel_bytes_full = static_cast<long long>(BN) * p.w_cols * 2;  // multiple of the chunk size (w_cols % 128 == 0)
    const long long n_chunks = (total_bytes + kFetchChunkBytes - 1) / kFetchChunkBytes;
    for (long long c = blockIdx.x; c < n_chunks; c += gridDim.x) {
      const long long byte0 = c * kFetchChunkBytes + fw * kFetchWarpBytes;
      // usually the warp's 16 KiB lie inside one owner's shard: resolve the owner once
      const long long last = min(byte0 + kFetchWarpBytes, total_bytes) - 1;
      const int owner0 = static_cast<int>(byte0 / shard_bytes);
      const bool one_owner = byte0 < total_bytes && owner0 == static_cast<int>(last / shard_bytes);
      const unsigned char* src0 = one_owner
          ? reinterpret_cast<const unsigned char*>(p.shard_ptrs[owner0]) - static_cast<long long>(owner0) * shard_bytes
          : nullptr;
      uint4 r[16];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int v = 0; v < 16; ++v) {
          const long long b = byte0 + (static_cast<long long>(half * 16 + v) * 32 + lane) * 16;
          if (b < total_bytes) {
            if (one_owner) {
              r[v] = ld_stream_v4(src0 + b);
            } else {
              const int owner = static_cast<int>(b / shard_bytes);
              r[v] = ld_stream_v4(reinterpret_cast<const unsigned char*>(p.shard_ptrs[owner]) + (b - owner * shard_bytes));
            }
          }
        }
#pragma unroll
        for (int v = 0; v < 16; ++v) {
          const long long b = byte0 + (static_cast<long long>(half * 16 + v) * 32 + lane) * 16;
          if (b < total_bytes) *reinterpret_cast<uint4*>(p.b_local + b) = r[v];
        }
      }
      __threadfence();
      __syncwarp();
      if (lane == 0) {
        const int panel = static_cast<int>((c * kFetchChunkBytes) / panel_bytes_full);
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.panel_flags + panel) : "memory");
      }
    }
  } else if (warp >= 2 && warp < 2 + Roles<kMode>::kEpilogueWarps) {
    // ------------------------------------------------------------------ epilogue
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) belong to this warp
    constexpr int kColGroups = Roles<kMode>::kEpilogueWarps / 4;   // warps sharing a lane quadrant split the columns
    const int col_group = (warp - 2) / 4;
    uint32_t local_tile = 0;
    uint32_t box_ctr = 0;  // output boxes staged so far by this CTA (selects the staging buffer)
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
      if constexpr (kMode != kModeScatter) {
        // Output through shared memory and the TMA unit: each 128-byte piece of an output row is written to a
        // swizzled staging box, and one thread stores (or reduce-adds) the whole 128-row box.  Rows and columns
        // outside the matrix are clipped by the tensor map.
        const int cols_per_box = p.c_is_f32 ? 32 : 64;
        const int n_boxes = BN / cols_per_box;
        const int my_row = quad * 32 + lane;
#pragma unroll 1
        for (int bx = 0; bx < n_boxes; ++bx) {
          uint32_t r[64];
          tmem_ld_32x32(t_row + bx * cols_per_box, r);
          if (!p.c_is_f32) tmem_ld_32x32(t_row + bx * cols_per_box + 32, r + 32);
          tmem_ld_wait();
          const int col0 = n0 + bx * cols_per_box;
          if (col0 >= p.N) continue;
          if constexpr (kMode == kModeScatterTma) {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * p.scale);
          }
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 64; ++i)
              if (i < cols_per_box && col0 + i < p.N)
                r[i] = __float_as_uint(__uint_as_float(r[i]) + __bfloat162float(p.bias[col0 + i]));
          }
          const int buf = static_cast<int>(box_ctr & 1u);
          const uint32_t use = box_ctr >> 1;
          if (use >= 1) {
            if (!(ok = mbar_wait(sfree0 + 8 * buf, (use - 1) & 1, wc, 6))) break;
          }
          uint8_t* srow = staging + buf * kStagingBytes + my_row * 128;
          if (p.c_is_f32) {
#pragma unroll
            for (int v = 0; v < 8; ++v)
              *reinterpret_cast<uint4*>(srow + ((v ^ (my_row & 7)) << 4)) =
                  make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
          } else {
            const __nv_bfloat16* rrow = (p.residual != nullptr && row_ok)
                                            ? p.residual + static_cast<long long>(row) * p.ldr + col0 : nullptr;
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(r[8 * v + i]);
              if (rrow != nullptr && col0 + 8 * v < p.N) {
                const uint4 res = *reinterpret_cast<const uint4*>(rrow + 8 * v);
                const uint32_t o[4] = {res.x, res.y, res.z, res.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  f[2 * i] += __uint_as_float(o[i] << 16);
                  f[2 * i + 1] += __uint_as_float(o[i] & 0xffff0000u);
                }
              }
              *reinterpret_cast<uint4*>(srow + ((v ^ (my_row & 7)) << 4)) =
                  make_uint4(pack2(f[0], f[1]), pack2(f[2], f[3]), pack2(f[4], f[5]), pack2(f[6], f[7]));
            }
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(sready0 + 8 * buf);
          if (warp == 2 && lane == 0) {
            if (mbar_wait(sready0 + 8 * buf, use & 1, wc, 7)) {
              if constexpr (kMode == kModeScatterTma) {
                // tiles never straddle owners (rows_per_rank is a multiple of the tile height)
                const int owner = m0 / p.rows_per_rank;
                tma_reduce_add_2d(&owners.m[owner], staging_u32 + buf * kStagingBytes, col0,
                                  m0 - owner * p.rows_per_rank);
              } else if (p.accumulate) {
                tma_reduce_add_2d(&tmap_c, staging_u32 + buf * kStagingBytes, col0, m0);
              } else {
                tma_store_2d(&tmap_c, staging_u32 + buf * kStagingBytes, col0, m0);
              }
              bulk_commit_group();
              if (box_ctr >= 1) {
                bulk_wait_group_read1();             // the previous box has been read: its buffer is free again
                mbar_arrive(sfree0 + 8 * (buf ^ 1));
              }
            }
          }
          ++box_ctr;
        }
        if (!ok) break;
      } else {
#pragma unroll 1
      for (int c = col_group * (BN / 32 / kColGroups); c < (col_group + 1) * (BN / 32 / kColGroups); ++c) {
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
        if constexpr (kMode == kModeScatter) {
          if (row_ok) {
            const int owner = row / p.rows_per_rank;
            float* dst = reinterpret_cast<float*>(p.acc_ptrs[owner]) + p.acc_offset +
                         static_cast<long long>(row - owner * p.rows_per_rank) * p.ldc + col0;
#pragma unroll
            for (int v = 0; v < 8; ++v)
              if (col0 + v * 4 < p.N)
                red_add_v4_f32(dst + 4 * v, f[4 * v] * p.scale, f[4 * v + 1] * p.scale, f[4 * v + 2] * p.scale,
                               f[4 * v + 3] * p.scale);
          }
        } else if (row_ok) {
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
            const __nv_bfloat16* rrow =
                p.residual ? p.residual + static_cast<long long>(row) * p.ldr + col0 : nullptr;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (col0 + v * 8 < p.N) {
                if (rrow != nullptr) {
                  const uint4 res = *reinterpret_cast<const uint4*>(rrow + 8 * v);
                  const uint32_t o[4] = {res.x, res.y, res.z, res.w};
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    f[8 * v + 2 * i] += __uint_as_float(o[i] << 16);
                    f[8 * v + 2 * i + 1] += __uint_as_float(o[i] & 0xffff0000u);
                  }
                }
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
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
    }
    if constexpr (kMode == kModeScatter) __threadfence_system();  // this thread's remote reductions are out
    if (kMode != kModeScatter && warp == 2 && lane == 0) {
      bulk_wait_group0();  // all output boxes are in memory
      if constexpr (kMode == kModeScatterTma) __threadfence_system();
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if constexpr (kMode == kModeScatter || kMode == kModeScatterTma) {
    // last CTA to finish releases one arrival on every owner's counter
    if (threadIdx.x == 0) {
      __threadfence_system();
      const unsigned int prev = atomicAdd(p.done_slot, 1u);
      if (prev == gridDim.x - 1) {
        *p.done_slot = 0;
        __threadfence_system();
        // A partial sum must never be counted as a contribution: no arrival if ANY CTA of this launch gave up
        // (each one records that in the global status word before it leaves), not only this last one.
        const bool clean = !*abort_flag && (p.status == nullptr || *reinterpret_cast<volatile int*>(p.status) == 0);
        if (clean)
          for (int r = 0; r < p.nranks; ++r)
            signal_add_release_sys(reinterpret_cast<unsigned long long*>(p.ctr_ptrs[r]), 1ull);
      }
    }
  }
}


}  // namespace gemm_impl
}  // namespace odc
