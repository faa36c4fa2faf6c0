// Causal attention over packed variable-length sequences on tcgen05 tensor cores (sm_100a).
//
// Forward: one CTA per (128 query rows of one sequence, query head).
//   warp 0     TMA producer: Q tile once, then K/V tiles of 128 keys through a small ring
//   warp 1     MMA issuer:   S = Q K^T into one of two TMEM buffers, then O += P V
//   warps 2-5  softmax:      one query row per thread; S from TMEM, online softmax in base 2 with
//                            lazy rescaling of O (only when a row maximum grows by more than 2^8),
//                            P written to shared memory as a 128-byte-swizzled bf16 operand
// S(j+1) is issued before P(j) is consumed, so the tensor core computes the next score tile while
// the softmax warps work on the current one.  K and V tiles share one TMA box shape: K is read as
// a K-major operand (Q K^T) and V as an N-major operand (P V), so nothing is transposed in memory.
// Rows/keys outside the sequence are masked; grouped-query attention maps query head h to
// key/value head h / (Hq/Hkv).
//
// Backward: a pre-pass computes delta = rowsum(dO * O); the main kernel owns one (128 keys, kv
// head) tile, keeps dK and dV in TMEM across all query tiles and query heads of the group, and
// recomputes P from the saved log-sum-exp.  dQ tiles are staged in shared memory as fp32 and added into a
// global fp32 buffer by the TMA unit (bulk reduce-add), then converted to bf16 by a post-pass.
//
// The reference calls flash-attn 2 for this op (examples/llm_training/torch_fsdp2.py:85-103).
#include <cuda.h>
#include <cuda_bf16.h>

#include <mutex>

#include "api.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"

namespace odc {

using namespace sm100;

namespace {

constexpr int kBlockQ = 128, kBlockKV = 128;
constexpr uint64_t kWaitBudgetNs = 4000000000ull;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.0f;

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// byte offset of element (row, col) inside a [128 rows][128 cols] bf16 operand stored as two
// 128-byte-swizzled slabs of 64 columns (the layout TMA produces and the K-major descriptor reads)
__device__ __forceinline__ uint32_t swz_chunk_offset(int row, int chunk16 /*0..15*/) {
  const int slab = chunk16 >> 3, ch = chunk16 & 7;
  return slab * 16384 + row * 128 + ((ch ^ (row & 7)) << 4);
}

struct FwdParams {
  const int* cu_seqlens;
  int num_seqs;
  int n_q, n_kv;
  __nv_bfloat16* o;
  long long o_stride;
  float* lse;  // [n_q, total_tokens]
  int total_tokens;
  float scale_log2;
  int causal;
  int* status;
};

// find (sequence, query block) of a linear block index; returns false if out of range
__device__ __forceinline__ bool locate_block(const int* cu, int num_seqs, int blk, int block_rows, int* seq,
                                             int* start, int* len, int* q0) {
  int acc = 0;
  for (int s = 0; s < num_seqs; ++s) {
    const int b = cu[s], e = cu[s + 1];
    const int nb = (e - b + block_rows - 1) / block_rows;
    if (blk < acc + nb) {
      *seq = s; *start = b; *len = e - b; *q0 = (blk - acc) * block_rows;
      return true;
    }
    acc += nb;
  }
  return false;
}

template <int D>
struct FwdCfg {
  // D = 64: one score buffer, 256 TMEM columns and 112 KiB of shared memory, so two CTAs share an SM
  // and hide each other's latency chains (most tiles of short sequences see only 1-3 key blocks).
  // D = 128: two score buffers, one CTA per SM.
  static constexpr int kStages = 2;
  static constexpr int kSBufs = (D == 64) ? 1 : 2;
  static constexpr int kTmemCols = (D == 64) ? 256 : 512;
  static constexpr int kOCol = kSBufs * 128;
  static constexpr int kCtasPerSm = (D == 64) ? 2 : 1;
  static constexpr int kQBytes = kBlockQ * D * 2;
  static constexpr int kKBytes = kBlockKV * D * 2;
  static constexpr int kStageBytes = 2 * kKBytes;
  static constexpr int kPBytes = kBlockQ * kBlockKV * 2;
  // barriers take 128 bytes; the alignment slack is trimmed for D = 64 so that two CTAs fit in one SM's
  // 228 KiB (the dynamic window starts 1024-byte aligned in practice; the kernel checks and reports otherwise)
  static constexpr int kAlignSlack = (D == 64) ? 768 : 1024;
  static constexpr int kSmem = kQBytes + kStages * kStageBytes + kPBytes + 128 + kAlignSlack;
};

template <int D>
__global__ void __launch_bounds__(192, FwdCfg<D>::kCtasPerSm)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const FwdParams p) {
  using C = FwdCfg<D>;
  int seq, seq_start, seq_len, q0;
  if (!locate_block(p.cu_seqlens, p.num_seqs, blockIdx.x, kBlockQ, &seq, &seq_start, &seq_len, &q0)) return;
  const int head = blockIdx.y;
  const int kv_head = head / (p.n_q / p.n_kv);
  const int kv_end = p.causal ? min(seq_len, q0 + kBlockQ) : seq_len;
  const int n_blocks = (kv_end + kBlockKV - 1) / kBlockKV;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  if (base - raw > static_cast<uint32_t>(C::kAlignSlack)) {  // cannot happen with a 1024-aligned window
    if (threadIdx.x == 0) report(p.status, kErrBounds, 40, static_cast<int>(base - raw));
    return;
  }
  const uint32_t q_smem = base;
  const uint32_t kv_smem = q_smem + C::kQBytes;
  const uint32_t p_smem = kv_smem + C::kStages * C::kStageBytes;
  uint8_t* p_ptr = smem + C::kQBytes + C::kStages * C::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_ptr + C::kPBytes);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t q_full = bar0;
  const uint32_t kv_full0 = bar0 + 8;                      // [kStages]
  const uint32_t kv_empty0 = kv_full0 + 8 * C::kStages;    // [kStages]
  const uint32_t s_full0 = kv_empty0 + 8 * C::kStages;     // [2]
  const uint32_t s_empty0 = s_full0 + 16;                  // [2]
  const uint32_t p_full = s_empty0 + 16;
  const uint32_t p_empty = p_full + 8;
  const uint32_t o_ready = p_empty + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::kStages + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitCtx wc{abort_flag, p.status, kWaitBudgetNs};

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(kv_full0 + 8 * s, 1);
      mbar_init(kv_empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_full0 + 8 * b, 1);
      mbar_init(s_empty0 + 8 * b, 4);
    }
    mbar_init(p_full, 4);
    mbar_init(p_empty, 1);
    mbar_init(o_ready, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s0 = tmem_base, tmem_o = tmem_base + C::kOCol;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v);
      mbar_arrive_expect_tx(q_full, C::kQBytes);
#pragma unroll
      for (int s = 0; s < D / 64; ++s) tma_load_2d(q_smem + s * 16384, &tmap_q, q_full, head * D + 64 * s, seq_start + q0);
      bool ok = true;
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int st = j % C::kStages;
        const uint32_t ph = (j / C::kStages) & 1;
        if (!(ok = mbar_wait(kv_empty0 + 8 * st, ph ^ 1, wc, 11))) break;
        const uint32_t bar = kv_full0 + 8 * st;
        mbar_arrive_expect_tx(bar, C::kStageBytes);
        const uint32_t k_dst = kv_smem + st * C::kStageBytes, v_dst = k_dst + C::kKBytes;
        const int row = seq_start + j * kBlockKV;
#pragma unroll
        for (int s = 0; s < D / 64; ++s) {
          tma_load_2d(k_dst + s * 16384, &tmap_k, bar, kv_head * D + 64 * s, row);
          tma_load_2d(v_dst + s * 16384, &tmap_v, bar, kv_head * D + 64 * s, row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(kBlockQ, kBlockKV, false, false);
      const uint32_t idesc_o = make_idesc_bf16(kBlockQ, D, false, true);
      bool ok = mbar_wait(q_full, 0, wc, 12);
      auto issue_s = [&](int j) {
        const int st = j % C::kStages;
        const uint32_t k_src = kv_smem + st * C::kStageBytes;
        const uint32_t d = tmem_s0 + (j % C::kSBufs) * 128;
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_f16(d, make_smem_desc(q_smem + off, 16, 1024), make_smem_desc(k_src + off, 16, 1024), idesc_s,
                   k > 0 ? 1u : 0u);
        }
        umma_commit(s_full0 + 8 * (j % C::kSBufs));
      };
      // S(j+1) may overwrite its buffer once the softmax of block j+1-kSBufs has read it
      auto issue_next_s = [&](int j) -> bool {
        if (j + 1 >= n_blocks) return true;
        const int st1 = (j + 1) % C::kStages;
        if (!mbar_wait(kv_full0 + 8 * st1, ((j + 1) / C::kStages) & 1, wc, 14)) return false;
        const int use = (j + 1) / C::kSBufs;
        if (use >= 1 && !mbar_wait(s_empty0 + 8 * ((j + 1) % C::kSBufs), (use - 1) & 1, wc, 15)) return false;
        tc_fence_after();
        issue_s(j + 1);
        return true;
      };
      if (ok && n_blocks > 0) {
        ok = mbar_wait(kv_full0, 0, wc, 13);
        if (ok) { tc_fence_after(); issue_s(0); }
      }
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (C::kSBufs == 2) {  // the next score tile runs while the softmax warps work on this one
          if (!(ok = issue_next_s(j))) break;
        }
        if (!(ok = mbar_wait(p_full, j & 1, wc, 16))) break;
        tc_fence_after();
        if (C::kSBufs == 1) {  // single buffer: free as soon as P(j) exists; queue S(j+1) ahead of P V(j)
          if (!(ok = issue_next_s(j))) break;
        }
        const int st = j % C::kStages;
        const uint32_t v_src = kv_smem + st * C::kStageBytes + C::kKBytes;
#pragma unroll
        for (int k = 0; k < kBlockKV / 16; ++k) {
          const uint64_t da = make_smem_desc(p_smem + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024);
          const uint64_t db = make_smem_desc(v_src + k * 2048, 16384, 1024);
          umma_f16(tmem_o, da, db, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(kv_empty0 + 8 * st);
        umma_commit(p_empty);
        umma_commit(o_ready);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue
    const int quad = warp & 3;
    const int row = quad * 32 + lane;            // query row within the tile
    const int q_rel = q0 + row;                  // position inside the sequence
    const bool row_valid = q_rel < seq_len;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_blocks && ok; ++j) {
      if (!(ok = mbar_wait(s_full0 + 8 * (j % C::kSBufs), (j / C::kSBufs) & 1, wc, 17))) break;
      tc_fence_after();
      const uint32_t t_s = tmem_s0 + (j % C::kSBufs) * 128 + lane_sel;
      const int kv0 = j * kBlockKV;
      const bool need_mask = (kv0 + kBlockKV > seq_len) || (p.causal && kv0 + kBlockKV > q0);
      // the whole score row (128 fp32) goes to registers with one wait; max, exp and packing run from there
      uint32_t sr[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32(t_s + c * 32, sr + c * 32);
      tmem_ld_wait();
      // four independent chains for the row maximum (and for the row sum below): a single running value would put
      // 128 dependent operations on the critical path of every key block
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      if (need_mask) {
        // keys [kv0, kv_hi) are visible to this row; everything from kv_hi on is masked
        const int kv_hi = min(seq_len, p.causal ? q_rel + 1 : seq_len) - kv0;
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          if (i >= kv_hi) sr[i] = 0xff800000u;  // -inf
          mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sr[i]));
        }
      } else {
#pragma unroll
        for (int i = 0; i < 128; ++i) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sr[i]));
      }
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      const float m_new = fmaxf(m_used, mx * p.scale_log2);
      // lazy rescale of the running output (exact: P and l keep using m_used until it is bumped)
      const bool bump = (m_new - m_used > kRescaleThreshold) || (m_used == -INFINITY && m_new > -INFINITY);
      if (j == 0) {
        m_used = m_new;
      } else if (__any_sync(0xffffffffu, bump)) {
        if (!(ok = mbar_wait(o_ready, (j - 1) & 1, wc, 18))) break;
        tc_fence_after();
        const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m_used - m_new);
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_o + lane_sel + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x16(tmem_o + lane_sel + c * 32, r);
          tmem_st_32x16(tmem_o + lane_sel + c * 32 + 16, r + 16);
        }
        tmem_st_wait();
        l *= alpha;
        m_used = m_new;
      }
      // P may be overwritten once the previous P V has finished reading it
      if (j > 0) {
        if (!(ok = mbar_wait(p_empty, (j - 1) & 1, wc, 19))) break;
      }
      const float m_sub = (m_used == -INFINITY) ? 0.f : m_used;
      float sum4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int v = 0; v < 16; ++v) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          f[i] = exp2f(fmaf(__uint_as_float(sr[8 * v + i]), p.scale_log2, -m_sub));
          sum4[i & 3] += f[i];
        }
        uint4 o;
        o.x = pack2(f[0], f[1]);
        o.y = pack2(f[2], f[3]);
        o.z = pack2(f[4], f[5]);
        o.w = pack2(f[6], f[7]);
        *reinterpret_cast<uint4*>(p_ptr + swz_chunk_offset(row, v)) = o;
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      // S buffer free for block j+2; P visible to the tensor core (async proxy)
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(s_empty0 + 8 * (j % C::kSBufs));
        mbar_arrive(p_full);
      }
    }
    // epilogue: O / l -> bf16, log-sum-exp
    if (ok && n_blocks > 0) ok = mbar_wait(o_ready, (n_blocks - 1) & 1, wc, 20);
    if (ok) {
      tc_fence_after();
      const float inv = (l > 0.f) ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.o + static_cast<long long>(seq_start + q_rel) * p.o_stride + head * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        if (n_blocks > 0) {
          tmem_ld_32x32(tmem_o + lane_sel + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0;
        }
        if (row_valid) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack2(__uint_as_float(r[8 * v]) * inv, __uint_as_float(r[8 * v + 1]) * inv);
            o.y = pack2(__uint_as_float(r[8 * v + 2]) * inv, __uint_as_float(r[8 * v + 3]) * inv);
            o.z = pack2(__uint_as_float(r[8 * v + 4]) * inv, __uint_as_float(r[8 * v + 5]) * inv);
            o.w = pack2(__uint_as_float(r[8 * v + 6]) * inv, __uint_as_float(r[8 * v + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) = o;
          }
        }
      }
      if (row_valid)
        p.lse[static_cast<long long>(head) * p.total_tokens + seq_start + q_rel] =
            (l > 0.f) ? (m_used + log2f(l)) * kLn2 : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}


// =================================================================================== backward
struct BwdParams {
  const int* cu_seqlens;
  int num_seqs;
  int n_q, n_kv;
  const float* lse;    // [n_q, total_tokens]
  const float* delta;  // [n_q, total_tokens]
  float* dq_acc;       // [total_tokens, n_q, D] fp32, zero-initialised
  __nv_bfloat16* dk;   // rows of n_kv * D values, dkv_stride elements apart
  __nv_bfloat16* dv;
  long long dkv_stride;
  int total_tokens;
  float scale, scale_log2;
  int causal;
  int* status;
};

template <int D>
struct BwdCfg {
  static constexpr int kStages = (D == 64) ? 2 : 1;
  static constexpr int kTile = 128 * D * 2;            // one [128][D] bf16 operand
  static constexpr int kStageBytes = 2 * kTile;        // Q_i and dO_i
  static constexpr int kPBytes = 128 * 128 * 2;
  // fp32 staging tile for the dQ reduction: D = 64 has room for its own 32 KiB, so the next P/dS can be written
  // while the TMA unit still reads it; D = 128 reuses the (consumed) P and dS buffers
  static constexpr int kDqStageBytes = (D == 64) ? 128 * 64 * 4 : 0;
  static constexpr int kSmem = 2 * kTile + kStages * kStageBytes + 2 * kPBytes + kDqStageBytes + 1024 + 256;
};

__device__ __forceinline__ void red_add_v4_gpu(float* p, float a, float b, float c, float d) {
  asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

constexpr int kBwdThreads = 32 * (2 + 8);  // TMA warp, MMA warp, two compute warpgroups (each takes half of the columns)

template <int D>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                const __grid_constant__ CUtensorMap tmap_dq, const BwdParams p) {
  using C = BwdCfg<D>;
  int seq, seq_start, seq_len, kv0;
  if (!locate_block(p.cu_seqlens, p.num_seqs, blockIdx.x, 128, &seq, &seq_start, &seq_len, &kv0)) return;
  const int kv_head = blockIdx.y;
  const int rep = p.n_q / p.n_kv;
  const int n_qblocks = (seq_len + 127) / 128;
  const int i_first = p.causal ? kv0 / 128 : 0;
  const int iters_per_head = n_qblocks - i_first;
  const int total_iters = iters_per_head * rep;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t k_smem = base, v_smem = base + C::kTile;
  const uint32_t ring = v_smem + C::kTile;
  const uint32_t p_smem = ring + C::kStages * C::kStageBytes;
  const uint32_t ds_smem = p_smem + C::kPBytes;
  uint8_t* p_ptr = smem + 2 * C::kTile + C::kStages * C::kStageBytes;
  uint8_t* ds_ptr = p_ptr + C::kPBytes;
  constexpr bool kOwnStage = C::kDqStageBytes > 0;
  uint8_t* stage_ptr = kOwnStage ? ds_ptr + C::kPBytes : p_ptr;
  const uint32_t stage_smem = kOwnStage ? ds_smem + C::kPBytes : p_smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ds_ptr + C::kPBytes + C::kDqStageBytes);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t kv_full = bar0;
  const uint32_t qdo_full0 = bar0 + 8;                      // [kStages]
  const uint32_t qdo_empty0 = qdo_full0 + 8 * C::kStages;   // [kStages]
  const uint32_t sdp_full = qdo_empty0 + 8 * C::kStages;
  const uint32_t pds_full = sdp_full + 8;
  const uint32_t dq_full = pds_full + 8;
  const uint32_t dq_read = dq_full + 8;
  const uint32_t dkv_full = dq_read + 8;
  const uint32_t stg_ready = dkv_full + 8;  // dQ staging tile written by all compute warps
  const uint32_t stg_free = stg_ready + 8;  // TMA has finished reading the staging tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::kStages + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const WaitCtx wc{abort_flag, p.status, kWaitBudgetNs};

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(qdo_full0 + 8 * s, 1);
      mbar_init(qdo_empty0 + 8 * s, 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 8);
    mbar_init(dq_full, 1);
    mbar_init(dq_read, 8);
    mbar_init(dkv_full, 1);
    mbar_init(stg_ready, 8);
    mbar_init(stg_free, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128, tm_dv = tmem_base + 256, tm_dk = tmem_base + 256 + D;
  // D = 64 leaves room for a private dQ tile, so the next S/dP can be issued while dQ is read out;
  // D = 128 fills all 512 columns and dQ_i reuses the score columns once the scores have been consumed
  constexpr bool kPrivateDq = (D == 64);
  const uint32_t tm_dq = kPrivateDq ? tmem_base + 384 : tm_s;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tmap_q); prefetch_tmap(&tmap_k); prefetch_tmap(&tmap_v); prefetch_tmap(&tmap_do);
      prefetch_tmap(&tmap_dq);
      mbar_arrive_expect_tx(kv_full, 2 * C::kTile);
#pragma unroll
      for (int s = 0; s < D / 64; ++s) {
        tma_load_2d(k_smem + s * 16384, &tmap_k, kv_full, kv_head * D + 64 * s, seq_start + kv0);
        tma_load_2d(v_smem + s * 16384, &tmap_v, kv_full, kv_head * D + 64 * s, seq_start + kv0);
      }
      bool ok = true;
      for (int it = 0; it < total_iters && ok; ++it) {
        const int head = kv_head * rep + it / iters_per_head;
        const int i = i_first + it % iters_per_head;
        const int st = it % C::kStages;
        if (!(ok = mbar_wait(qdo_empty0 + 8 * st, ((it / C::kStages) & 1) ^ 1, wc, 31))) break;
        const uint32_t bar = qdo_full0 + 8 * st;
        mbar_arrive_expect_tx(bar, C::kStageBytes);
        const uint32_t q_dst = ring + st * C::kStageBytes, do_dst = q_dst + C::kTile;
        const int row = seq_start + i * 128;
#pragma unroll
        for (int s = 0; s < D / 64; ++s) {
          tma_load_2d(q_dst + s * 16384, &tmap_q, bar, head * D + 64 * s, row);
          tma_load_2d(do_dst + s * 16384, &tmap_do, bar, head * D + 64 * s, row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);   // S, dP: both operands K-major
      const uint32_t idesc_tt = make_idesc_bf16(128, D, true, true);      // dV, dK: A^T (MN-major) x MN-major
      const uint32_t idesc_dq = make_idesc_bf16(128, D, false, true);     // dQ: K-major x MN-major
      bool ok = mbar_wait(kv_full, 0, wc, 32);
      for (int it = 0; it < total_iters && ok; ++it) {
        const int st = it % C::kStages;
        const uint32_t q_src = ring + st * C::kStageBytes, do_src = q_src + C::kTile;
        if (!(ok = mbar_wait(qdo_full0 + 8 * st, (it / C::kStages) & 1, wc, 33))) break;
        if (!kPrivateDq && it > 0) {  // the score columns still hold dQ of the previous tile until it has been read out
          if (!(ok = mbar_wait(dq_read, (it - 1) & 1, wc, 34))) break;
        }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_f16(tm_s, make_smem_desc(q_src + off, 16, 1024), make_smem_desc(k_smem + off, 16, 1024), idesc_s,
                   k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t off = (k >> 2) * 16384 + (k & 3) * 32;
          umma_f16(tm_dp, make_smem_desc(do_src + off, 16, 1024), make_smem_desc(v_smem + off, 16, 1024), idesc_s,
                   k > 0 ? 1u : 0u);
        }
        umma_commit(sdp_full);
        if (!(ok = mbar_wait(pds_full, it & 1, wc, 35))) break;
        tc_fence_after();
        // dV += P^T dO ; dK += dS^T Q   (reduction over the 128 query rows, 16 at a time)
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          umma_f16(tm_dv, make_smem_desc(p_smem + k * 2048, 16384, 1024), make_smem_desc(do_src + k * 2048, 16384, 1024),
                   idesc_tt, (it > 0 || k > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          umma_f16(tm_dk, make_smem_desc(ds_smem + k * 2048, 16384, 1024), make_smem_desc(q_src + k * 2048, 16384, 1024),
                   idesc_tt, (it > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(qdo_empty0 + 8 * st);  // Q_i / dO_i are not read again: their stage can be refilled now
        // dQ_i = dS K   (reduction over the 128 keys)
        if (kPrivateDq && it > 0) {  // the private dQ tile of the previous query tile must have been read out
          if (!(ok = mbar_wait(dq_read, (it - 1) & 1, wc, 34))) break;
          tc_fence_after();
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          umma_f16(tm_dq, make_smem_desc(ds_smem + (k >> 2) * 16384 + (k & 3) * 32, 16, 1024),
                   make_smem_desc(k_smem + k * 2048, 16384, 1024), idesc_dq, k > 0 ? 1u : 0u);
        }
        umma_commit(dq_full);
      }
      if (ok) umma_commit(dkv_full);
    }
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;            // which 64 of the 128 key columns this warpgroup handles
    const int row = quad * 32 + lane;
    const uint32_t lane_sel = static_cast<uint32_t>(quad * 32) << 16;
    bool ok = true;
    for (int it = 0; it < total_iters && ok; ++it) {
      const int head = kv_head * rep + it / iters_per_head;
      const int i = i_first + it % iters_per_head;
      const int q_rel = i * 128 + row;
      const bool q_valid = q_rel < seq_len;
      const long long tok = seq_start + q_rel;
      const float lse2 = q_valid ? p.lse[static_cast<long long>(head) * p.total_tokens + tok] * kLog2e : 0.f;
      const float dlt = q_valid ? p.delta[static_cast<long long>(head) * p.total_tokens + tok] : 0.f;
      if (!(ok = mbar_wait(sdp_full, it & 1, wc, 36))) break;
      tc_fence_after();
      // the P/dS buffers double as the staging tile of the previous dQ reduction: wait until TMA has read it
      if (!kOwnStage && it > 0) {
        if (!(ok = mbar_wait(stg_free, (it - 1) & 1, wc, 39))) break;
      }
      uint32_t rs[64], rd[64];
      tmem_ld_32x32(tm_s + lane_sel + half * 64, rs);
      tmem_ld_32x32(tm_s + lane_sel + half * 64 + 32, rs + 32);
      tmem_ld_32x32(tm_dp + lane_sel + half * 64, rd);
      tmem_ld_32x32(tm_dp + lane_sel + half * 64 + 32, rd + 32);
      tmem_ld_wait();
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        float pf[8], df[8];
#pragma unroll
        for (int x = 0; x < 8; ++x) {
          const int col = half * 64 + v * 8 + x;
          const int kv = kv0 + col;
          const bool okk = q_valid && kv < seq_len && (!p.causal || kv <= q_rel);
          const float pv = okk ? exp2f(fmaf(__uint_as_float(rs[v * 8 + x]), p.scale_log2, -lse2)) : 0.f;
          pf[x] = pv;
          df[x] = pv * (__uint_as_float(rd[v * 8 + x]) - dlt) * p.scale;
        }
        uint4 a, b;
        a.x = pack2(pf[0], pf[1]); a.y = pack2(pf[2], pf[3]); a.z = pack2(pf[4], pf[5]); a.w = pack2(pf[6], pf[7]);
        b.x = pack2(df[0], df[1]); b.y = pack2(df[2], df[3]); b.z = pack2(df[4], df[5]); b.w = pack2(df[6], df[7]);
        const uint32_t off = swz_chunk_offset(row, half * 8 + v);
        *reinterpret_cast<uint4*>(p_ptr + off) = a;
        *reinterpret_cast<uint4*>(ds_ptr + off) = b;
      }
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      // dQ tile -> fp32 staging in shared memory (over the consumed P/dS buffers) -> TMA reduce-add into the
      // global accumulator; rows past the end of the sequence are staged as zeros
      if (!(ok = mbar_wait(dq_full, it & 1, wc, 37))) break;
      tc_fence_after();
      if (kOwnStage && it > 0) {  // the private staging tile of the previous query tile must have been read
        if (!(ok = mbar_wait(stg_free, (it - 1) & 1, wc, 39))) break;
      }
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(tm_dq + lane_sel + half * (D / 2) + c * 32, r);
        tmem_ld_wait();
        const int box = half * (D / 64) + c;
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          uint4 o = q_valid ? make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]) : make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(stage_ptr + box * 16384 + row * 128 + ((v ^ (row & 7)) << 4)) = o;
        }
      }
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(stg_ready);
        mbar_arrive(dq_read);
      }
      if (warp == 2 && lane == 0) {  // one thread hands the staged tile to the TMA unit and frees it once read
        if (mbar_wait(stg_ready, it & 1, wc, 40)) {
#pragma unroll
          for (int b2 = 0; b2 < D / 32; ++b2)
            tma_reduce_add_2d(&tmap_dq, stage_smem + b2 * 16384, head * D + 32 * b2, seq_start + i * 128);
          bulk_commit_group();
          bulk_wait_group_read0();
        }
        mbar_arrive(stg_free);
      }
      __syncwarp();
    }
    if (warp == 2 && lane == 0) bulk_wait_group0();
    // dK / dV of this key tile: one warpgroup writes dV, the other dK
    if (ok) ok = mbar_wait(dkv_full, 0, wc, 38);
    if (ok) {
      tc_fence_after();
      const int kv_rel = kv0 + row;
      const bool kv_valid = kv_rel < seq_len;
      const long long off = static_cast<long long>(seq_start + kv_rel) * p.dkv_stride + kv_head * D;
      __nv_bfloat16* dst = (half == 0 ? p.dv : p.dk) + off;
      const uint32_t src = (half == 0 ? tm_dv : tm_dk) + lane_sel;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        if (total_iters > 0) {
          tmem_ld_32x32(src + c * 32, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int x = 0; x < 32; ++x) r[x] = 0;
        }
        if (kv_valid) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 o;
            o.x = pack2(__uint_as_float(r[8 * v]), __uint_as_float(r[8 * v + 1]));
            o.y = pack2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
            o.z = pack2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
            o.w = pack2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
            *reinterpret_cast<uint4*>(dst + c * 32 + v * 8) = o;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// delta[h, t] = sum_d dO[t, h, d] * O[t, h, d].  A thread takes 16 bytes of both tensors; the D/8 threads of one
// (token, head) pair are neighbours in a warp and combine with shuffles.  A CTA covers 256 / (D/8) consecutive
// tokens and walks the heads, so the loads of a warp are whole 128-byte rows and the stores of one head form one
// contiguous run of tokens.
template <int D>
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ o, float* __restrict__ delta,
                  int total_tokens, int n_q, long long do_stride, long long o_stride) {
  constexpr int kLanes = D / 8;               // threads per (token, head)
  constexpr int kTokens = 256 / kLanes;       // tokens per CTA
  const int part = threadIdx.x % kLanes;
  const int t = blockIdx.x * kTokens + threadIdx.x / kLanes;
  const bool live = t < total_tokens;
  const __nv_bfloat16* a = dout + static_cast<long long>(live ? t : 0) * do_stride + part * 8;
  const __nv_bfloat16* b = o + static_cast<long long>(live ? t : 0) * o_stride + part * 8;
  for (int h = 0; h < n_q; ++h) {
    float s = 0.f;
    if (live) {
      const uint4 x = *reinterpret_cast<const uint4*>(a + h * D);
      const uint4 y = *reinterpret_cast<const uint4*>(b + h * D);
      const uint32_t xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {y.x, y.y, y.z, y.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s += __uint_as_float(xs[i] << 16) * __uint_as_float(ys[i] << 16);
        s += __uint_as_float(xs[i] & 0xffff0000u) * __uint_as_float(ys[i] & 0xffff0000u);
      }
    }
#pragma unroll
    for (int off = kLanes / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (live && part == 0) delta[static_cast<long long>(h) * total_tokens + t] = s;
  }
}

// acc is dense [tokens, width] fp32; dq rows are dq_stride elements apart
__global__ void __launch_bounds__(256)
cast_dq_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long n8, int width8,
               long long dq_stride) {
  for (long long v = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; v < n8;
       v += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 a = *reinterpret_cast<const float4*>(acc + v * 8);
    const float4 b = *reinterpret_cast<const float4*>(acc + v * 8 + 4);
    const long long row = v / width8;
    const int col = static_cast<int>(v % width8) * 8;
    *reinterpret_cast<uint4*>(dq + row * dq_stride + col) =
        make_uint4(pack2(a.x, a.y), pack2(a.z, a.w), pack2(b.x, b.y), pack2(b.z, b.w));
  }
}

}  // namespace

cudaError_t attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_seqlens,
                     int num_seqs, int total_tokens, int max_seqlen, int n_q, int n_kv, int head_dim,
                     long long q_stride, long long kv_stride, long long o_stride, float scale, bool causal,
                     int* status, int sm_count, cudaStream_t stream) {
  (void)max_seqlen;
  (void)sm_count;
  if (total_tokens == 0 || num_seqs == 0) return cudaSuccess;
  if (head_dim != 64 && head_dim != 128) return cudaErrorInvalidValue;
  if (n_q % n_kv != 0) return cudaErrorInvalidValue;
  if ((q_stride % 8) || (kv_stride % 8) || (o_stride % 8)) return cudaErrorInvalidValue;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(o)) & 15)
    return cudaErrorMisalignedAddress;
  CUtensorMap tq, tk, tv;
  if (!encode_tile_map_2d(&tq, q, static_cast<uint64_t>(n_q) * head_dim, total_tokens, q_stride * 2, 64, kBlockQ) ||
      !encode_tile_map_2d(&tk, k, static_cast<uint64_t>(n_kv) * head_dim, total_tokens, kv_stride * 2, 64, kBlockKV) ||
      !encode_tile_map_2d(&tv, v, static_cast<uint64_t>(n_kv) * head_dim, total_tokens, kv_stride * 2, 64, kBlockKV))
    return cudaErrorInvalidValue;
  FwdParams p;
  p.cu_seqlens = cu_seqlens; p.num_seqs = num_seqs; p.n_q = n_q; p.n_kv = n_kv;
  p.o = static_cast<__nv_bfloat16*>(o); p.o_stride = o_stride; p.lse = lse; p.total_tokens = total_tokens;
  p.scale_log2 = scale * kLog2e; p.causal = causal ? 1 : 0; p.status = status;
  const int blocks = (total_tokens + kBlockQ - 1) / kBlockQ + num_seqs;
  dim3 grid(blocks, n_q);
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(attn_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<64>::kSmem);
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(attn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      FwdCfg<128>::kSmem);
  });
  if (attr_err != cudaSuccess) return attr_err;
  if (head_dim == 64)
    attn_fwd_kernel<64><<<grid, 192, FwdCfg<64>::kSmem, stream>>>(tq, tk, tv, p);
  else
    attn_fwd_kernel<128><<<grid, 192, FwdCfg<128>::kSmem, stream>>>(tq, tk, tv, p);
  return cudaGetLastError();
}

}  // namespace odc

namespace odc {

cudaError_t attn_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o, const float* lse,
                     void* dq, void* dk, void* dv, float* delta, float* dq_acc, const int* cu_seqlens, int num_seqs,
                     int total_tokens, int max_seqlen, int n_q, int n_kv, int head_dim, long long q_stride,
                     long long kv_stride, long long o_stride, long long dq_stride, long long dkv_stride, float scale,
                     bool causal, int* status, int sm_count, cudaStream_t stream) {
  (void)max_seqlen;
  if (total_tokens == 0 || num_seqs == 0) return cudaSuccess;
  if (head_dim != 64 && head_dim != 128) return cudaErrorInvalidValue;
  if (n_q % n_kv != 0) return cudaErrorInvalidValue;
  if ((q_stride % 8) || (kv_stride % 8) || (o_stride % 8) || (dq_stride % 8) || (dkv_stride % 8))
    return cudaErrorInvalidValue;
  // dout is contiguous [T, n_q, D]; dq / dk / dv rows may be strided (views of one fused qkv gradient)
  const long long do_stride = static_cast<long long>(n_q) * head_dim;
  if (head_dim == 64) {
    attn_delta_kernel<64><<<(total_tokens + 31) / 32, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(o), delta, total_tokens, n_q,
        do_stride, o_stride);
  } else {
    attn_delta_kernel<128><<<(total_tokens + 15) / 16, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(dout), static_cast<const __nv_bfloat16*>(o), delta, total_tokens, n_q,
        do_stride, o_stride);
  }
  cudaError_t e = cudaMemsetAsync(dq_acc, 0, sizeof(float) * static_cast<size_t>(total_tokens) * n_q * head_dim, stream);
  if (e != cudaSuccess) return e;
  CUtensorMap tq, tk, tv, tdo, tdq;
  if (!encode_tile_map_2d_f32(&tdq, dq_acc, static_cast<uint64_t>(n_q) * head_dim, total_tokens,
                              static_cast<uint64_t>(n_q) * head_dim * 4, 32, 128))
    return cudaErrorInvalidValue;
  if (!encode_tile_map_2d(&tq, q, static_cast<uint64_t>(n_q) * head_dim, total_tokens, q_stride * 2, 64, 128) ||
      !encode_tile_map_2d(&tk, k, static_cast<uint64_t>(n_kv) * head_dim, total_tokens, kv_stride * 2, 64, 128) ||
      !encode_tile_map_2d(&tv, v, static_cast<uint64_t>(n_kv) * head_dim, total_tokens, kv_stride * 2, 64, 128) ||
      !encode_tile_map_2d(&tdo, dout, static_cast<uint64_t>(n_q) * head_dim, total_tokens, do_stride * 2, 64, 128))
    return cudaErrorInvalidValue;
  BwdParams p;
  p.cu_seqlens = cu_seqlens; p.num_seqs = num_seqs; p.n_q = n_q; p.n_kv = n_kv; p.lse = lse; p.delta = delta;
  p.dq_acc = dq_acc; p.dk = static_cast<__nv_bfloat16*>(dk); p.dv = static_cast<__nv_bfloat16*>(dv);
  p.total_tokens = total_tokens; p.scale = scale; p.scale_log2 = scale * kLog2e; p.causal = causal ? 1 : 0;
  p.status = status; p.dkv_stride = dkv_stride;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(attn_bwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdCfg<64>::kSmem);
    if (attr_err == cudaSuccess)
      attr_err = cudaFuncSetAttribute(attn_bwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      BwdCfg<128>::kSmem);
  });
  if (attr_err != cudaSuccess) return attr_err;
  dim3 grid((total_tokens + 127) / 128 + num_seqs, n_kv);
  if (head_dim == 64)
    attn_bwd_kernel<64><<<grid, kBwdThreads, BwdCfg<64>::kSmem, stream>>>(tq, tk, tv, tdo, tdq, p);
  else
    attn_bwd_kernel<128><<<grid, kBwdThreads, BwdCfg<128>::kSmem, stream>>>(tq, tk, tv, tdo, tdq, p);
  const long long n8 = static_cast<long long>(total_tokens) * n_q * head_dim / 8;
  long long g = (n8 + 255) / 256;
  if (g > sm_count * 16) g = sm_count * 16;
  cast_dq_kernel<<<static_cast<int>(g), 256, 0, stream>>>(dq_acc, static_cast<__nv_bfloat16*>(dq), n8,
                                                          n_q * head_dim / 8, dq_stride);
  return cudaGetLastError();
}

}  // namespace odc
