// bf16 GEMM on CTA pairs (tcgen05 cta_group::2) for sm_100a: one 256 x 256 output tile per pair of SMs.
//
// Two CTAs of a cluster work on one tile.  Each CTA stages ITS half of the A tile (128 rows) and ITS half of the B
// tile (128 rows of B, i.e. 128 output columns) with ordinary per-CTA TMA loads, and holds the accumulator rows
// of its A half (128 lanes x 256 fp32 columns) in its own tensor memory.  One thread of the even CTA (the leader)
// issues tcgen05.mma.cta_group::2: the tensor cores of both SMs read both halves of B, so every byte of B is
// fetched from L2 and written to shared memory once per PAIR instead of once per SM, and a stage of the ring is
// 32 KiB per CTA instead of 48 KiB (six stages instead of four).
//
//   warp 0      : TMA producer of this CTA's halves; byte counts are reported to the leader's "full" barrier
//   warp 1      : leader only: MMA issuer; completion is committed to BOTH CTAs' barriers (two commits, no multicast)
//   warps 2..5  : epilogue of this CTA's 128 rows (tcgen05.ld -> bias / residual -> swizzled staging -> TMA store),
//                 then a (remote) arrive on the leader's "accumulator free" barrier
// Two accumulators (all 512 TMEM columns of each CTA) alternate, so the epilogue of one tile overlaps the main
// loop of the next.  Every copy in this file is an ordinary per-CTA TMA copy into that CTA's own shared memory.  Every wait is bounded and reports through the
// status word; a pair whose partner gave up runs into its own bounded waits and leaves the same way.
//
// Operand layouts, edge handling and the epilogue are those of the single-CTA kernel (gemm_tcgen05.cu).
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdlib.h>

#include <mutex>

#include "api.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"

namespace odc {
namespace gemm_pair {

using namespace sm100;

constexpr int BMH = 128, BNH = 128, BN = 256, BK = 64;   // per-CTA halves; the pair's tile is 256 x 256
constexpr int kStages = 6;
constexpr int kATile = BMH * BK * 2;                     // 16 KiB
constexpr int kBTile = BNH * BK * 2;                     // 16 KiB
constexpr int kStageBytes = kATile + kBTile;             // 32 KiB per CTA
constexpr int kStagingBytes = 128 * 128;
constexpr int kSmemBytes = kStages * kStageBytes + 2 * kStagingBytes + 1024 + 256;
constexpr uint32_t kTmemCols = 512;
constexpr uint64_t kWaitBudgetNs = 4000000000ull;
constexpr int kThreads = 192;

struct Params {
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  long long ldr;
  int M, N, K;
  int c_is_f32, accumulate;
  int a_mn, b_mn;
  int tiles_m, tiles_n;   // in units of the pair's 256 x 256 tile
  int* status;
  // kModeScatter: the epilogue adds every 128-row output box into the fp32 accumulator of the rank that owns those rows
  const long long* ctr_ptrs;   // [nranks] arrival counters
  int rows_per_rank;           // output rows owned by one rank (a multiple of 128)
  int nranks;
  float scale;
  unsigned int* done_slot;     // self-resetting CTA completion counter
  // kModeGather: operand B (a row-sharded weight) is assembled from the owners' shards while the GEMM runs
  const long long* shard_ptrs; // [nranks] base address of each owner's [rows_per_rank, w_cols] bf16 shard
  unsigned char* b_local;      // local [w_rows, w_cols] bf16 buffer the shards are gathered into (tensor map B covers it)
  unsigned int* panel_flags;   // [ceil(w_rows / 256)] chunks landed per 256-row group (zeroed before the launch)
  int w_rows, w_cols;          // gathered matrix: [N, K] when B is K-major (y = x W^T), [K, N] when MN-major (dx = dy W)
  // Rotation of the work order by this rank's position in the group.  Without it every rank would pull the first
  // owner's rows first (and push into the first owner's accumulator first): one GPU's links saturated, seven idle.
  // Each rank starts at the rows it owns itself and walks the owners from there, like the stand-alone kernels do.
  int rot_m, rot_n;            // tile rows / tile columns by which the tile order is rotated
  int rot_kb;                  // k-blocks by which the k loop is rotated (gathered reduction dimension)
  long long fetch_rot;         // 64 KiB chunks by which the fetch order is rotated
};

constexpr int kModePlain = 0, kModeScatter = 1, kModeGather = 2;
constexpr int kFetchWarps = 4;
constexpr int kFetchWarpBytes = 16384;                  // moved by one fetch warp between two flag updates
constexpr int kFetchChunkBytes = kFetchWarps * kFetchWarpBytes;
template <int kMode> struct Roles {
  static constexpr int kThreadsTotal = kThreads + (kMode == kModeGather ? 32 * kFetchWarps : 0);
};
constexpr int kMaxOwners = 8;
struct OwnerMaps {   // one fp32 tensor map per owner's accumulator region (kModeScatter)
  CUtensorMap m[kMaxOwners];
};

// Tile order: groups of kGroupM tile rows are walked column by column (rows fastest inside a group), so the pairs
// that run at the same time share a few A row panels and a few B column panels and both stay in L2 however large
// the whole operands are.
constexpr int kGroupM = 16;
__device__ __forceinline__ void tile_coords(int tile, const Params& p, int* tm, int* tn) {
  const int per_group = kGroupM * p.tiles_n;
  const int group = tile / per_group;
  const int first_m = group * kGroupM;
  const int gsize = min(p.tiles_m - first_m, kGroupM);
  const int in_group = tile - group * per_group;
  int m = first_m + in_group % gsize + p.rot_m;
  int n = in_group / gsize + p.rot_n;
  *tm = m >= p.tiles_m ? m - p.tiles_m : m;
  *tn = n >= p.tiles_n ? n - p.tiles_n : n;
}

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int kMode>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Roles<kMode>::kThreadsTotal, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ OwnerMaps owners,
                      const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  uint8_t* staging = smem + kStages * kStageBytes;
  const uint32_t staging_u32 = base + kStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 2 * kStagingBytes);
  const uint32_t full0 = smem_u32(bars);                    // [kStages]  used in the leader: both CTAs' bytes landed
  const uint32_t empty0 = full0 + 8 * kStages;              // [kStages]  per CTA: the MMAs have read this stage
  const uint32_t tfull0 = empty0 + 8 * kStages;             // [2]        per CTA: accumulator complete
  const uint32_t tempty0 = tfull0 + 16;                     // [2]        used in the leader: both epilogues drained it
  const uint32_t sready0 = tempty0 + 16;                    // [2]
  const uint32_t sfree0 = sready0 + 16;                     // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();                   // 0: leader
  const WaitCtx wc{abort_flag, p.status, kWaitBudgetNs};

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8 * a, 1);
      mbar_init(tempty0 + 8 * a, 8);   // four epilogue warps in each CTA of the pair
      mbar_init(sready0 + 8 * a, 4);
      mbar_init(sfree0 + 8 * a, 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the partner's barriers exist before anything is reported to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.tiles_m * p.tiles_n;
  const int k_blocks = (p.K + BK - 1) / BK;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      prefetch_tmap(&tmap_a);
      prefetch_tmap(&tmap_b);
      // gather mode: wait (bounded) until every chunk of 256-row group `g` of the gathered matrix is in local memory
      // groups already known complete: in address order a running count is enough (the reduction dimension is
      // walked front to back); a rotated walk keeps a bitmask of the first 512 groups (later ones are re-checked)
      int groups_ready = 0;
      uint32_t ready[16] = {0};
      const bool rotated = p.rot_kb != 0 || p.rot_n != 0;
      auto wait_group = [&](int g) -> bool {
        if (!rotated) {
          if (g < groups_ready) return true;
        } else if (g < 512 && ((ready[g >> 5] >> (g & 31)) & 1u)) {
          return true;
        }
        const long long group_bytes = static_cast<long long>(min(BN, p.w_rows - g * BN)) * p.w_cols * 2;
        const unsigned int target =
            static_cast<unsigned int>((group_bytes + kFetchChunkBytes - 1) / kFetchChunkBytes) * kFetchWarps;
        const uint64_t t0 = globaltimer_ns();
        unsigned int seen;
        while (true) {
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(p.panel_flags + g) : "memory");
          if (seen >= target) break;
          if (*abort_flag) return false;
          if (globaltimer_ns() - t0 > kWaitBudgetNs) {
            *abort_flag = 1;
            report(p.status, kErrPipelineTimeout, 25, g);
            return false;
          }
          __nanosleep(64);
        }
        asm volatile("fence.proxy.async;" ::: "memory");  // generic-proxy stores -> visible to TMA reads
        if (!rotated) {
          if (p.b_mn) groups_ready = g + 1;
        } else if (g < 512) {
          ready[g >> 5] |= 1u << (g & 31);
        }
        return true;
      };
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        int tm, tn;
        tile_coords(tile, p, &tm, &tn);
        const int m0 = tm * 256 + static_cast<int>(cta) * BMH;   // this CTA's rows of A and C
        const int n0 = tn * BN + static_cast<int>(cta) * BNH;    // this CTA's rows of B
        if constexpr (kMode == kModeGather) {
          // B K-major (forward): the 256 weight rows this tile multiplies must have landed in local memory first
          if (!p.b_mn && !(ok = wait_group(tn))) break;
        }
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if constexpr (kMode == kModeGather) {
            // B MN-major (input gradient): the gathered rows are the reduction dimension, 4 k-blocks per group
            if (p.b_mn && !(ok = wait_group(((p.rot_kb ? (kb + p.rot_kb) % k_blocks : kb) * BK) / BN))) break;
          }
          if (!(ok = mbar_wait(empty0 + 8 * s, ph ^ 1, wc, 11))) break;
          const uint32_t sa = base + s * kStageBytes;
          const uint32_t sb = sa + kATile;
          if (cta == 0) mbar_arrive_expect_tx(full0 + 8 * s, 2 * kStageBytes);   // bytes of both CTAs
          const uint32_t bar = mapa_shared(full0 + 8 * s, 0);
          const int k0 = (p.rot_kb ? (kb + p.rot_kb) % k_blocks : kb) * BK;
          if (!p.a_mn) {
            tma_load_2d_pair(sa, &tmap_a, bar, k0, m0);                 // box {64 k, 128 rows}
          } else {
#pragma unroll
            for (int i = 0; i < BMH / 64; ++i) tma_load_2d_pair(sa + i * 8192, &tmap_a, bar, m0 + 64 * i, k0);
          }
          if (!p.b_mn) {
            tma_load_2d_pair(sb, &tmap_b, bar, k0, n0);                 // box {64 k, 128 rows}
          } else {
#pragma unroll
            for (int i = 0; i < BNH / 64; ++i) tma_load_2d_pair(sb + i * 8192, &tmap_b, bar, n0 + 64 * i, k0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (lane == 0 && cta == 0) {
      const uint32_t idesc = make_idesc_bf16(256, 256, p.a_mn != 0, p.b_mn != 0);
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
      const uint32_t a_kstep = p.a_mn ? 2048u : 32u, b_kstep = p.b_mn ? 2048u : 32u;  // bytes per K = 16
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local_tile) {
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!(ok = mbar_wait(tempty0 + 8 * acc, acc_ph ^ 1, wc, 12))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          if (!(ok = mbar_wait(full0 + 8 * s, ph, wc, 13))) break;
          tc_fence_after();
          const uint32_t sa = base + s * kStageBytes;
          const uint32_t sb = sa + kATile;
#pragma unroll
          for (int j = 0; j < BK / 16; ++j) {
            const uint64_t da = make_smem_desc(sa + j * a_kstep, a_lbo, 1024);
            const uint64_t db = make_smem_desc(sb + j * b_kstep, b_lbo, 1024);
            umma_f16_pair(d_tmem, da, db, idesc, (kb > 0 || j > 0) ? 1u : 0u);
          }
          // the stage is reusable in BOTH CTAs once these MMAs have read it
          umma_commit_pair(mapa_shared(empty0 + 8 * s, 0));
          umma_commit_pair(mapa_shared(empty0 + 8 * s, 1));
        }
        if (ok) {
          umma_commit_pair(mapa_shared(tfull0 + 8 * acc, 0));
          umma_commit_pair(mapa_shared(tfull0 + 8 * acc, 1));
        }
      }
    }
  } else if (kMode == kModeGather && warp >= 6) {
    // ------------------------------------------------------------------ shard fetch (every CTA of the grid)
    // The owners' shards are copied into the local B buffer in address order (= group order): 64 KiB per step and
    // CTA, 16 KiB per warp with 16 x 16-byte peer loads in flight per lane; after its part a warp makes the stores
    // visible and counts them on the group's flag.
    const int fw = warp - 6;
    const long long total_bytes = static_cast<long long>(p.w_rows) * p.w_cols * 2;
    const long long shard_bytes = static_cast<long long>(p.rows_per_rank) * p.w_cols * 2;
    const long long panel_bytes_full = static_cast<long long>(BN) * p.w_cols * 2;  // a multiple of the chunk size
    const long long n_chunks = (total_bytes + kFetchChunkBytes - 1) / kFetchChunkBytes;
    for (long long c0 = blockIdx.x; c0 < n_chunks; c0 += gridDim.x) {
      // rotated: this rank's own rows first, then the next owner's, ...
      const long long c = p.fetch_rot ? (c0 + p.fetch_rot) % n_chunks : c0;
      const long long byte0 = c * kFetchChunkBytes + fw * kFetchWarpBytes;
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
  } else if (warp >= 2 && warp < 6) {
    // ------------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad+32) belong to this warp
    uint32_t local_tile = 0;
    uint32_t box_ctr = 0;
    bool ok = true;
    const uint32_t tempty_leader0 = mapa_shared(tempty0, 0);
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local_tile) {
      int tm, tn;
      tile_coords(tile, p, &tm, &tn);
      const int m0 = tm * 256 + static_cast<int>(cta) * BMH;
      const int n0 = tn * BN;
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      if (!(ok = mbar_wait(tfull0 + 8 * acc, acc_ph, wc, 14))) break;
      tc_fence_after();
      const int my_row = quad * 32 + lane;
      const int row = m0 + my_row;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + acc * BN;
      const int cols_per_box = p.c_is_f32 ? 32 : 64;
      const int n_boxes = BN / cols_per_box;
#pragma unroll 1
      for (int bx = 0; bx < n_boxes; ++bx) {
        uint32_t r[64];
        tmem_ld_32x32(t_row + bx * cols_per_box, r);
        if (!p.c_is_f32) tmem_ld_32x32(t_row + bx * cols_per_box + 32, r + 32);
        tmem_ld_wait();
        const int col0 = n0 + bx * cols_per_box;
        if (col0 >= p.N || m0 >= p.M) continue;
        if constexpr (kMode == kModeScatter) {
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
          if (!(ok = mbar_wait(sfree0 + 8 * buf, (use - 1) & 1, wc, 16))) break;
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
          if (mbar_wait(sready0 + 8 * buf, use & 1, wc, 17)) {
            if constexpr (kMode == kModeScatter) {
              // a CTA's 128 rows never straddle two owners (rows_per_rank is a multiple of 128)
              const int owner = m0 / p.rows_per_rank;
              tma_reduce_add_2d(&owners.m[owner], staging_u32 + buf * kStagingBytes, col0, m0 - owner * p.rows_per_rank);
            } else if (p.accumulate) {
              tma_reduce_add_2d(&tmap_c, staging_u32 + buf * kStagingBytes, col0, m0);
            } else {
              tma_store_2d(&tmap_c, staging_u32 + buf * kStagingBytes, col0, m0);
            }
            bulk_commit_group();
            if (box_ctr >= 1) {
              bulk_wait_group_read1();
              mbar_arrive(sfree0 + 8 * (buf ^ 1));
            }
          }
        }
        ++box_ctr;
      }
      if (!ok) break;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader0 + 8 * acc);   // the leader may overwrite this accumulator
    }
    if (warp == 2 && lane == 0) {
      bulk_wait_group0();  // all output boxes are in memory
      if constexpr (kMode == kModeScatter) __threadfence_system();
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // nothing is reported to the partner's barriers, or read from its shared memory, after this
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if constexpr (kMode == kModeScatter) {
    // the last CTA to finish releases one arrival on every owner's counter, unless any CTA of the launch gave up
    if (threadIdx.x == 0) {
      __threadfence_system();
      const unsigned int prev = atomicAdd(p.done_slot, 1u);
      if (prev == gridDim.x - 1) {
        *p.done_slot = 0;
        __threadfence_system();
        const bool clean = !*abort_flag && (p.status == nullptr || *reinterpret_cast<volatile int*>(p.status) == 0);
        if (clean)
          for (int r = 0; r < p.nranks; ++r)
            signal_add_release_sys(reinterpret_cast<unsigned long long*>(p.ctr_ptrs[r]), 1ull);
      }
    }
  }
}

}  // namespace gemm_pair

// ODC_GEMM_ROTATE: 0 (default) every rank walks the owners in address order; 1: the forward gather and the
// weight-gradient scatter start at the rank's own rows and walk the owners from there; 2: the input-gradient
// gather (rotated k loop) as well.  Measured on 8 GPUs with all ranks launching the same kernel at once, rotation
// makes the forward kernels faster (0.863 -> 0.799 ms and 1.247 -> 0.766 ms on the two widest weights) and the
// input-gradient kernel slower; a whole training step, where ranks are not in lock-step anyway, measured slower with
// it, so it is off unless asked for.
static int rotate_mode() {
  static const int mode = [] {
    const char* e = getenv("ODC_GEMM_ROTATE");
    return e == nullptr ? 0 : atoi(e);
  }();
  return mode;
}

// Returns cudaErrorNotSupported when the shape is not worth a CTA pair (the caller then uses the single-CTA kernel).
cudaError_t gemm_bf16_pair(const void* a, const void* b, void* c, int c_kind, const void* bias, int M, int N, int K,
                           int layout, bool accumulate, long long lda, long long ldb, long long ldc, int* status,
                           int sm_count, cudaStream_t stream, const void* residual, long long ldr) {
  using namespace gemm_pair;
  if (M < 256 || N < 256 || K < BK || sm_count < 2) return cudaErrorNotSupported;
  const bool a_mn = (layout == 2);
  const bool b_mn = (layout != 0);
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c)) & 15)
    return cudaErrorMisalignedAddress;
  if ((lda % 8) || (ldb % 8) || (N % 8) || (ldc % (c_kind == kF32 ? 4 : 8))) return cudaErrorInvalidDevicePointer;
  if (c_kind != kF32 && accumulate) return cudaErrorNotSupported;

  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_bf16_pair_kernel<kModePlain>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSmemBytes);
  });
  if (attr_err != cudaSuccess) return attr_err;

  CUtensorMap ta, tb, tc;
  if (!a_mn) {
    if (!encode_tile_map_2d(&ta, a, K, M, lda * 2, 64, BMH)) return cudaErrorInvalidPitchValue;
  } else {
    if (!encode_tile_map_2d(&ta, a, M, K, lda * 2, 64, 64)) return cudaErrorInvalidPitchValue;
  }
  if (!b_mn) {
    if (!encode_tile_map_2d(&tb, b, K, N, ldb * 2, 64, BNH)) return cudaErrorInvalidTexture;
  } else {
    if (!encode_tile_map_2d(&tb, b, N, K, ldb * 2, 64, 64)) return cudaErrorInvalidTexture;
  }
  if (c_kind == kF32) {
    if (!encode_tile_map_2d_f32(&tc, c, N, M, ldc * 4, 32, BMH)) return cudaErrorInvalidValue;
  } else {
    if (!encode_tile_map_2d(&tc, c, N, M, ldc * 2, 64, BMH)) return cudaErrorInvalidValue;
  }
  Params p{};
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.M = M; p.N = N; p.K = K;
  p.c_is_f32 = (c_kind == kF32);
  p.accumulate = accumulate ? 1 : 0;
  p.a_mn = a_mn; p.b_mn = b_mn;
  p.tiles_m = (M + 255) / 256;
  p.tiles_n = (N + BN - 1) / BN;
  p.status = status;
  if (residual != nullptr) {
    if (c_kind != kBF16 || (ldr % 8) || (reinterpret_cast<uintptr_t>(residual) & 15)) return cudaErrorInvalidValue;
    p.residual = static_cast<const __nv_bfloat16*>(residual);
    p.ldr = ldr;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int pairs = tiles < sm_count / 2 ? tiles : sm_count / 2;
  gemm_bf16_pair_kernel<kModePlain><<<2 * pairs, kThreads, kSmemBytes, stream>>>(ta, tb, tc, OwnerMaps{}, p);
  return cudaGetLastError();
}

// dW[n_out, k_in] = dY^T X on CTA pairs; every 128 x 32 fp32 output box is added (x scale) into the accumulator of the
// rank that owns its rows by the TMA unit, through the peer mapping; then one arrival per owner.  Same contract as
// gemm_wgrad_scatter_tma; returns cudaErrorNotSupported for shapes it does not take.
cudaError_t gemm_wgrad_scatter_pair(const void* dy, const void* x, int tokens, int n_out, int k_in, long long ld_dy,
                                    long long ld_x, const long long* acc_addrs_host, const long long* ctr_ptrs,
                                    long long acc_offset, int rows_per_rank, int nranks, float scale,
                                    unsigned int* done_slot, int* status, int sm_count, cudaStream_t stream,
                                    int start_rank) {
  using namespace gemm_pair;
  if (n_out < 256 || k_in < 256 || tokens < BK || sm_count < 2) return cudaErrorNotSupported;
  if (nranks > kMaxOwners || (rows_per_rank % BMH) != 0) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(dy) | reinterpret_cast<uintptr_t>(x)) & 15) return cudaErrorMisalignedAddress;
  if ((ld_dy % 8) || (ld_x % 8) || (k_in % 8) || (acc_offset % 4)) return cudaErrorInvalidValue;
  if (static_cast<long long>(rows_per_rank) * nranks < n_out) return cudaErrorInvalidValue;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_bf16_pair_kernel<kModeScatter>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSmemBytes);
  });
  if (attr_err != cudaSuccess) return attr_err;
  CUtensorMap ta, tb;
  // "tn": A = dY viewed as [K = tokens rows, M = n_out cols], B = X as [K = tokens rows, N = k_in cols]
  if (!encode_tile_map_2d(&ta, dy, n_out, tokens, ld_dy * 2, 64, 64)) return cudaErrorInvalidValue;
  if (!encode_tile_map_2d(&tb, x, k_in, tokens, ld_x * 2, 64, 64)) return cudaErrorInvalidValue;
  OwnerMaps owners{};
  for (int r = 0; r < nranks; ++r) {
    float* base = reinterpret_cast<float*>(static_cast<uintptr_t>(acc_addrs_host[r])) + acc_offset;
    if (!encode_tile_map_2d_f32(&owners.m[r], base, k_in, rows_per_rank, static_cast<uint64_t>(k_in) * 4, 32, BMH))
      return cudaErrorInvalidValue;
  }
  Params p{};
  p.M = n_out; p.N = k_in; p.K = tokens;
  p.c_is_f32 = 1;
  p.a_mn = 1; p.b_mn = 1;
  p.tiles_m = (n_out + 255) / 256;
  p.tiles_n = (k_in + BN - 1) / BN;
  p.status = status;
  p.ctr_ptrs = ctr_ptrs;
  p.rows_per_rank = rows_per_rank; p.nranks = nranks; p.scale = scale; p.done_slot = done_slot;
  if (rotate_mode() >= 1)
    p.rot_m = static_cast<int>((static_cast<long long>(start_rank) * rows_per_rank / 256) % p.tiles_m);
  const int tiles = p.tiles_m * p.tiles_n;
  const int pairs = tiles < sm_count / 2 ? tiles : sm_count / 2;
  gemm_bf16_pair_kernel<kModeScatter><<<2 * pairs, kThreads, kSmemBytes, stream>>>(ta, tb, ta, owners, p);
  return cudaGetLastError();
}

// Y[M, N] = X[M, K] W[N, K]^T (dgrad = false) or dX[M, K_in] = dY[M, N_out] W[N_out, K_in] (dgrad = true) on CTA pairs,
// with W row-sharded over nranks owners and pulled into w_local by four extra warps per CTA while the GEMM runs.
// Same contracts as gemm_gather_nt / gemm_gather_nn; cudaErrorNotSupported for shapes it does not take.
cudaError_t gemm_gather_pair(bool dgrad, const void* a, const long long* shard_ptrs, void* w_local, void* out,
                             const void* bias, int M, int w_rows, int w_cols, long long lda, long long ldo,
                             int rows_per_rank, int nranks, unsigned int* group_flags, int* status, int sm_count,
                             cudaStream_t stream, const void* residual, long long ldr, int start_rank) {
  using namespace gemm_pair;
  const int N = dgrad ? w_cols : w_rows;   // output columns
  const int K = dgrad ? w_rows : w_cols;   // reduction length
  if (M < 256 || N < 256 || K < BK || sm_count < 2) return cudaErrorNotSupported;
  if ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(w_local) | reinterpret_cast<uintptr_t>(out)) & 15)
    return cudaErrorMisalignedAddress;
  if ((lda % 8) || (ldo % 8) || (N % 8) || (w_cols % 128)) return cudaErrorInvalidValue;
  if (static_cast<long long>(rows_per_rank) * nranks < w_rows) return cudaErrorInvalidValue;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(gemm_bf16_pair_kernel<kModeGather>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    kSmemBytes);
  });
  if (attr_err != cudaSuccess) return attr_err;
  CUtensorMap ta, tb, tc;
  if (!encode_tile_map_2d(&ta, a, K, M, lda * 2, 64, BMH)) return cudaErrorInvalidValue;
  if (!dgrad) {
    if (!encode_tile_map_2d(&tb, w_local, w_cols, w_rows, static_cast<uint64_t>(w_cols) * 2, 64, BNH)) return cudaErrorInvalidValue;
  } else {  // B is MN-major: rows = reduction index, box {64 output columns, 64 reduction rows}
    if (!encode_tile_map_2d(&tb, w_local, w_cols, w_rows, static_cast<uint64_t>(w_cols) * 2, 64, 64)) return cudaErrorInvalidValue;
  }
  if (!encode_tile_map_2d(&tc, out, N, M, ldo * 2, 64, BMH)) return cudaErrorInvalidValue;
  Params p{};
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.M = M; p.N = N; p.K = K;
  p.b_mn = dgrad ? 1 : 0;
  p.tiles_m = (M + 255) / 256;
  p.tiles_n = (N + BN - 1) / BN;
  p.status = status;
  p.shard_ptrs = shard_ptrs;
  p.b_local = static_cast<unsigned char*>(w_local);
  p.panel_flags = group_flags;
  p.rows_per_rank = rows_per_rank; p.nranks = nranks;
  p.w_rows = w_rows; p.w_cols = w_cols;
  if (rotate_mode() >= (dgrad ? 2 : 1)) {
    const int groups = (w_rows + BN - 1) / BN;
    const int rot_group = static_cast<int>((static_cast<long long>(start_rank) * rows_per_rank / BN) % groups);
    if (!dgrad) p.rot_n = rot_group % p.tiles_n;
    else p.rot_kb = (rot_group * (BN / BK)) % ((K + BK - 1) / BK);
    p.fetch_rot = static_cast<long long>(rot_group) * (static_cast<long long>(BN) * w_cols * 2 / kFetchChunkBytes);
  }
  if (residual != nullptr) {
    if ((ldr % 8) || (reinterpret_cast<uintptr_t>(residual) & 15)) return cudaErrorInvalidValue;
    p.residual = static_cast<const __nv_bfloat16*>(residual);
    p.ldr = ldr;
  }
  cudaError_t e = cudaMemsetAsync(group_flags, 0, sizeof(unsigned int) * ((w_rows + BN - 1) / BN), stream);
  if (e != cudaSuccess) return e;
  const int grid = sm_count & ~1;  // every CTA also fetches, so the whole machine runs even when there are few tiles
  gemm_bf16_pair_kernel<kModeGather><<<grid, Roles<kModeGather>::kThreadsTotal, kSmemBytes, stream>>>(ta, tb, tc, OwnerMaps{}, p);
  return cudaGetLastError();
}

}  // namespace odc
