// gather / scatter_accumulate / arrival wait: the two on-demand primitives as single launches.
//
// gather: CTAs are striped over (peer, tile) pairs, so all peers' links are busy at once; each
// thread keeps several 16-byte peer loads in flight and may narrow fp32 -> bf16 on the way.
// Replaces the reference's serial per-peer Tensor.copy_ plus separate cast
// (odc/primitives/gather.py:121-127, odc/fsdp/fsdp2.py:339-351).
//
// scatter_accumulate: rows of the local gradient go to their owners as 16-byte vector
// reductions into the fp32 accumulator (no mailbox, no second pass on the owner); the last CTA
// to finish bumps every owner's arrival counter with a system-scope release.  Replaces mailbox
// copy + request/ack kernels + watcher add (odc/primitives/scatter_accumulate.py:649-691,369-395).
#include <stdlib.h>

#include "api.h"
#include "odc_device.cuh"
#include "sm100_ptx.cuh"

namespace odc {

namespace {

constexpr int kThreads = 512;
constexpr int kVecPerThread = 4;                        // 16-byte accesses in flight per thread
constexpr size_t kTileVecs = size_t(kThreads) * kVecPerThread;  // 16-byte vectors per tile (32 KiB)

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

// ---------------------------------------------------------------- gather, same dtype ----------
// bytes-per-row copy; src rows are peers' buffers, dst rows are consecutive in `out`.
__global__ void __launch_bounds__(kThreads)
gather_copy_kernel(const long long* __restrict__ peers, unsigned char* __restrict__ out, size_t row_bytes,
                   int nranks, int start, int vec_ok, int check, int* status, size_t src_region_bytes) {
  if (check) {  // debug launch: refuse instead of faulting; every thread takes the same branch
    if (start < 0 || start >= nranks) {
      if (threadIdx.x == 0) report(status, kErrPeerIndex, start, nranks);
      return;
    }
    if (src_region_bytes != 0 && row_bytes > src_region_bytes) {  // would read past the registered shard
      if (threadIdx.x == 0) report(status, kErrBounds, -1, static_cast<int>(src_region_bytes / 16));
      return;
    }
    for (int p = 0; p < nranks; ++p) {
      if (peers[p] == 0 || (vec_ok && (peers[p] & 15) != 0)) {
        if (threadIdx.x == 0) report(status, kErrBounds, p, 0);
        return;
      }
    }
  }
  const size_t nvec = vec_ok ? row_bytes / 16 : 0;
  const size_t tiles_per_row = (nvec + kTileVecs - 1) / kTileVecs;
  const size_t total_tiles = tiles_per_row * nranks;
  for (size_t t = blockIdx.x; t < total_tiles; t += gridDim.x) {
    const int peer = (static_cast<int>(t % nranks) + start) % nranks;
    const size_t tile = t / nranks;
    const uint4* src = reinterpret_cast<const uint4*>(peers[peer]);
    uint4* dst = reinterpret_cast<uint4*>(out + size_t(peer) * row_bytes);
    const size_t v0 = tile * kTileVecs + threadIdx.x;
    uint4 r[kVecPerThread];
#pragma unroll
    for (int k = 0; k < kVecPerThread; ++k) {
      const size_t v = v0 + size_t(k) * kThreads;
      if (v < nvec) r[k] = ld_stream_v4(src + v);
    }
#pragma unroll
    for (int k = 0; k < kVecPerThread; ++k) {
      const size_t v = v0 + size_t(k) * kThreads;
      if (v < nvec) dst[v] = r[k];
    }
  }
  // bytes not covered by whole vectors (everything when rows are not 16-byte aligned)
  const size_t tail0 = nvec * 16;
  const size_t tail = row_bytes - tail0;
  const size_t total_tail = tail * nranks;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total_tail; i += size_t(gridDim.x) * blockDim.x) {
    const int p = static_cast<int>(i / tail);
    const size_t j = tail0 + i % tail;
    out[size_t(p) * row_bytes + j] = reinterpret_cast<const unsigned char*>(peers[p])[j];
  }
}

// ---------------------------------------------------------------- gather, fp32 -> bf16 --------
__global__ void __launch_bounds__(kThreads)
gather_f32_to_bf16_kernel(const long long* __restrict__ peers, __nv_bfloat16* __restrict__ out, size_t n,
                          int nranks, int start, int check, int* status, size_t src_region_elems) {
  if (check) {
    if (start < 0 || start >= nranks) {
      if (threadIdx.x == 0) report(status, kErrPeerIndex, start, nranks);
      return;
    }
    if (src_region_elems != 0 && n > src_region_elems) {
      if (threadIdx.x == 0) report(status, kErrBounds, -1, static_cast<int>(src_region_elems / 16));
      return;
    }
    for (int p = 0; p < nranks; ++p) {
      if (peers[p] == 0 || (peers[p] & 15) != 0) {
        if (threadIdx.x == 0) report(status, kErrBounds, p, 0);
        return;
      }
    }
  }
  const size_t nvec = n / 8;  // 8 floats in (2 x 16 B), 8 bf16 out (16 B)
  constexpr size_t kTile = size_t(kThreads) * 2;
  const size_t tiles_per_row = (nvec + kTile - 1) / kTile;
  const size_t total_tiles = tiles_per_row * nranks;
  const bool aligned = (n % 8) == 0;  // row starts stay 16-byte aligned in the output
  if (aligned) {
    for (size_t t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const int peer = (static_cast<int>(t % nranks) + start) % nranks;
      const size_t tile = t / nranks;
      const uint4* src = reinterpret_cast<const uint4*>(peers[peer]);
      uint4* dst = reinterpret_cast<uint4*>(out + size_t(peer) * n);
      uint4 a[2], b[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const size_t v = tile * kTile + threadIdx.x + size_t(k) * kThreads;
        if (v < nvec) {
          a[k] = ld_stream_v4(src + 2 * v);
          b[k] = ld_stream_v4(src + 2 * v + 1);
        }
      }
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const size_t v = tile * kTile + threadIdx.x + size_t(k) * kThreads;
        if (v < nvec) {
          uint4 o;
          o.x = pack_bf16x2(__uint_as_float(a[k].x), __uint_as_float(a[k].y));
          o.y = pack_bf16x2(__uint_as_float(a[k].z), __uint_as_float(a[k].w));
          o.z = pack_bf16x2(__uint_as_float(b[k].x), __uint_as_float(b[k].y));
          o.w = pack_bf16x2(__uint_as_float(b[k].z), __uint_as_float(b[k].w));
          dst[v] = o;
        }
      }
    }
  } else {
    const size_t total = n * nranks;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
      const int peer = static_cast<int>(i / n);
      const size_t j = i % n;
      out[i] = __float2bfloat16(reinterpret_cast<const float*>(peers[peer])[j]);
    }
  }
}

// ---------------------------------------------------------------- scatter-accumulate ---------
// Completion: every thread's reductions -> __threadfence_system -> block barrier -> one thread
// counts the CTA done; the last CTA releases one arrival on each owner's counter.
__device__ __forceinline__ void finish_and_signal(const long long* ctrs, int nranks, unsigned int* done_slot) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(done_slot, 1u);
    if (prev == gridDim.x - 1) {
      *done_slot = 0;  // self-reset: the slot is reusable by a later launch
      __threadfence_system();
      for (int p = 0; p < nranks; ++p)
        signal_add_release_sys(reinterpret_cast<unsigned long long*>(ctrs[p]), 1ull);
    }
  }
}

// Debug launch (acc_len != 0): `extent` elements starting at each owner's accumulator base must fit the declared
// accumulator length, the rotation start must name a member of the group and no table entry may be null or
// misaligned.  A refused launch touches no accumulator; it still signals arrival so that no owner waits for it, and
// the producer's host raises from the status word.  Uniform across the grid: every thread takes the same branch.
// Returns 0: proceed; 1: refused, counters usable (signal arrival); 2: refused, the tables themselves are bad.
__device__ __forceinline__ int scatter_refused(const long long* accs, const long long* ctrs, int nranks, int start,
                                               long long extent, long long acc_len, int* status) {
  if (acc_len == 0) return 0;
  int code = kOk, detail = 0, seen = 0;
  bool tables_ok = true;
  for (int p = 0; p < nranks; ++p)
    if (accs[p] == 0 || (accs[p] & 3) != 0 || ctrs[p] == 0 || (ctrs[p] & 7) != 0) {
      code = kErrBounds; detail = p; tables_ok = false; break;
    }
  if (!tables_ok) {
    if (threadIdx.x == 0 && blockIdx.x == 0) report(status, code, detail, seen);
    return 2;
  }
  if (start < 0 || start >= nranks) {
    code = kErrPeerIndex; detail = start; seen = nranks;
  } else if (extent > acc_len) {
    code = kErrBounds; detail = -1; seen = static_cast<int>(acc_len < 0x7fffffff ? acc_len : 0x7fffffff);
  }
  if (code == kOk) return 0;
  if (threadIdx.x == 0 && blockIdx.x == 0) report(status, code, detail, seen);
  return 1;
}

template <typename InT>
__global__ void __launch_bounds__(kThreads)
scatter_acc_f32_kernel(const InT* __restrict__ inp, const long long* __restrict__ accs,
                       const long long* __restrict__ ctrs, size_t n, int nranks, int start, float scale,
                       unsigned int* done_slot, int vec_ok, long long acc_len, int* status) {
  if (const int refused = scatter_refused(accs, ctrs, nranks, start, static_cast<long long>(n), acc_len, status)) {
    if (refused == 1) finish_and_signal(ctrs, nranks, done_slot);
    return;
  }
  constexpr int kPerVec = 4;  // one 16-byte reduction = 4 floats
  const size_t nvec = n / kPerVec;
  const bool aligned = vec_ok != 0;
  if (aligned) {
    const size_t tiles_per_row = (nvec + kTileVecs - 1) / kTileVecs;
    const size_t total_tiles = tiles_per_row * nranks;
    for (size_t t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const int peer = (static_cast<int>(t % nranks) + start) % nranks;
      const size_t tile = t / nranks;
      float* acc = reinterpret_cast<float*>(accs[peer]);
      const InT* row = inp + size_t(peer) * n;
      float4 r[kVecPerThread];
#pragma unroll
      for (int k = 0; k < kVecPerThread; ++k) {
        const size_t v = tile * kTileVecs + threadIdx.x + size_t(k) * kThreads;
        if (v < nvec) {
          if constexpr (sizeof(InT) == 4) {
            r[k] = *reinterpret_cast<const float4*>(row + v * 4);
          } else {
            const uint2 u = *reinterpret_cast<const uint2*>(row + v * 4);
            r[k] = make_float4(bf16_lo(u.x), bf16_hi(u.x), bf16_lo(u.y), bf16_hi(u.y));
          }
        }
      }
#pragma unroll
      for (int k = 0; k < kVecPerThread; ++k) {
        const size_t v = tile * kTileVecs + threadIdx.x + size_t(k) * kThreads;
        if (v < nvec) red_add_v4_f32(acc + v * 4, r[k].x * scale, r[k].y * scale, r[k].z * scale, r[k].w * scale);
      }
    }
    // tail of each row (n % 4 elements; only reachable with nranks == 1 here)
    if (blockIdx.x == 0) {
      for (size_t j = nvec * 4 + threadIdx.x; j < n; j += blockDim.x)
        for (int p = 0; p < nranks; ++p)
          red_add_f32(reinterpret_cast<float*>(accs[p]) + j, float(inp[size_t(p) * n + j]) * scale);
    }
  } else {
    const size_t total = n * nranks;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
      const int peer = static_cast<int>(i / n);
      red_add_f32(reinterpret_cast<float*>(accs[peer]) + (i % n), float(inp[i]) * scale);
    }
  }
  finish_and_signal(ctrs, nranks, done_slot);
}

// ---------------------------------------------------------------- scatter-accumulate, segmented
// The same reduction taken straight from a list of gradient tensors, with no flattened [owners, shard] staging
// copy in between.  Segment s is a contiguous tensor of `total` elements whose dim-0 chunk for owner r is
// [r * chunk, min((r + 1) * chunk, total)) (later owners may get fewer or no elements: padding); it is added at
// element `dst` of every owner's accumulator.  A tile is 4 * kTileVecs elements of one (segment, owner) pair.
template <typename InT>
__global__ void __launch_bounds__(kThreads)
scatter_acc_segments_kernel(const __grid_constant__ ScatterSegments segs, const long long* __restrict__ accs,
                            const long long* __restrict__ ctrs, int nranks, int start, float scale,
                            unsigned int* done_slot, long long acc_len, int* status) {
  {
    long long extent = 0;
    for (int s = 0; s < segs.count; ++s) extent = max(extent, segs.dst[s] + min(segs.chunk[s], segs.total[s]));
    if (const int refused = scatter_refused(accs, ctrs, nranks, start, extent, acc_len, status)) {
      if (refused == 1) finish_and_signal(ctrs, nranks, done_slot);
      return;
    }
  }
  constexpr long long kTileElems = static_cast<long long>(kTileVecs) * 4;
  const long long tiles_per_owner = segs.tile_prefix[segs.count];
  const long long total_tiles = tiles_per_owner * nranks;
  for (long long t = blockIdx.x; t < total_tiles; t += gridDim.x) {
    const int owner = (static_cast<int>(t % nranks) + start) % nranks;
    const long long q = t / nranks;
    int si = 0;
    while (si + 1 < segs.count && q >= segs.tile_prefix[si + 1]) ++si;
    const long long chunk = segs.chunk[si];
    const long long len = max(0ll, min(chunk, segs.total[si] - static_cast<long long>(owner) * chunk));
    const long long e0 = (q - segs.tile_prefix[si]) * kTileElems;
    if (e0 >= len) continue;
    const InT* src = static_cast<const InT*>(segs.src[si]) + static_cast<long long>(owner) * chunk;
    float* acc = reinterpret_cast<float*>(accs[owner]) + segs.dst[si];
    if (segs.vec[si]) {
      float4 r[kVecPerThread];
#pragma unroll
      for (int k = 0; k < kVecPerThread; ++k) {
        const long long e = e0 + (threadIdx.x + static_cast<long long>(k) * kThreads) * 4;
        if (e + 4 <= len) {
          if constexpr (sizeof(InT) == 4) {
            r[k] = *reinterpret_cast<const float4*>(src + e);
          } else {
            const uint2 u = *reinterpret_cast<const uint2*>(src + e);
            r[k] = make_float4(bf16_lo(u.x), bf16_hi(u.x), bf16_lo(u.y), bf16_hi(u.y));
          }
        }
      }
#pragma unroll
      for (int k = 0; k < kVecPerThread; ++k) {
        const long long e = e0 + (threadIdx.x + static_cast<long long>(k) * kThreads) * 4;
        if (e + 4 <= len) {
          red_add_v4_f32(acc + e, r[k].x * scale, r[k].y * scale, r[k].z * scale, r[k].w * scale);
        } else if (e < len) {  // ragged end of the last owner's chunk
          for (long long j = e; j < len; ++j) red_add_f32(acc + j, float(src[j]) * scale);
        }
      }
    } else {
      // a chunk or destination that is not 16-byte aligned: one element per reduction
      const long long e1 = min(len, e0 + kTileElems);
      for (long long j = e0 + threadIdx.x; j < e1; j += kThreads) red_add_f32(acc + j, float(src[j]) * scale);
    }
  }
  finish_and_signal(ctrs, nranks, done_slot);
}

// bf16 gradients into bf16 accumulators (accumulation_dtype left at the input dtype)
__global__ void __launch_bounds__(kThreads)
scatter_acc_bf16_kernel(const __nv_bfloat16* __restrict__ inp, const long long* __restrict__ accs,
                        const long long* __restrict__ ctrs, size_t n, int nranks, int start, float scale,
                        unsigned int* done_slot, long long acc_len, int* status) {
  if (const int refused = scatter_refused(accs, ctrs, nranks, start, static_cast<long long>(n), acc_len, status)) {
    if (refused == 1) finish_and_signal(ctrs, nranks, done_slot);
    return;
  }
  const bool aligned = (n % 2) == 0;
  const size_t total = n * nranks;
  if (aligned) {
    const size_t pairs = total / 2;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < pairs; i += size_t(gridDim.x) * blockDim.x) {
      const size_t e = i * 2;
      const int peer = (static_cast<int>(e / n) + start) % nranks;
      const size_t j = e % n;
      const uint32_t u = *reinterpret_cast<const uint32_t*>(inp + size_t(peer) * n + j);
      const uint32_t s = pack_bf16x2(bf16_lo(u) * scale, bf16_hi(u) * scale);
      red_add_bf16x2(reinterpret_cast<__nv_bfloat16*>(accs[peer]) + j, s);
    }
  } else {
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += size_t(gridDim.x) * blockDim.x) {
      const int peer = static_cast<int>(i / n);
      atomicAdd(reinterpret_cast<__nv_bfloat16*>(accs[peer]) + (i % n),
                __float2bfloat16(__bfloat162float(inp[i]) * scale));
    }
  }
  finish_and_signal(ctrs, nranks, done_slot);
}

// ---------------------------------------------------------------- scatter-accumulate, bulk (TMA) path ---------
// fp32 rows into fp32 accumulators without touching registers: one thread per CTA streams 32 KiB pieces
// global -> shared (bulk copy, mbarrier completion) and shared -> owner's accumulator (bulk reduce-add through
// the peer mapping).  Four pieces per CTA are in flight, i.e. ~19 MB across the GPU, which is what keeps the
// links busy; the SMs' load/store and atomic pipes stay idle.
constexpr int kBulkBytes = 32768;
constexpr int kBulkStages = 4;
constexpr int kBulkSmem = kBulkStages * kBulkBytes + 64;

__global__ void __launch_bounds__(32)
scatter_acc_bulk_kernel(const float* __restrict__ inp, const long long* __restrict__ accs,
                        const long long* __restrict__ ctrs, size_t n, int nranks, int start,
                        unsigned int* done_slot, int* status, long long acc_len) {
  extern __shared__ __align__(128) unsigned char bulk_smem[];
  using namespace sm100;
  __shared__ int abort_flag;
  if (const int refused = scatter_refused(accs, ctrs, nranks, start, static_cast<long long>(n), acc_len, status)) {
    if (refused == 1) finish_and_signal(ctrs, nranks, done_slot);
    return;
  }
  const uint32_t buf0 = smem_u32(bulk_smem);
  const uint32_t bar0 = buf0 + kBulkStages * kBulkBytes;
  const size_t row_bytes = n * sizeof(float);
  const size_t tiles_per_row = (row_bytes + kBulkBytes - 1) / kBulkBytes;
  const size_t total_tiles = tiles_per_row * nranks;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kBulkStages; ++s) mbar_init(bar0 + 8 * s, 1);
    fence_barrier_init();
    const WaitCtx wc{&abort_flag, status, 4000000000ull};
    auto tile_info = [&](size_t t, const float** src, float** dst, uint32_t* bytes) {
      const int peer = (static_cast<int>(t % nranks) + start) % nranks;
      const size_t off = (t / nranks) * kBulkBytes;
      const size_t len = row_bytes - off < size_t(kBulkBytes) ? row_bytes - off : size_t(kBulkBytes);
      *src = reinterpret_cast<const float*>(reinterpret_cast<const unsigned char*>(inp + size_t(peer) * n) + off);
      *dst = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(accs[peer]) + off);
      *bytes = static_cast<uint32_t>(len);
    };
    auto issue_load = [&](size_t t, int s) {
      const float* src; float* dst; uint32_t bytes;
      tile_info(t, &src, &dst, &bytes);
      mbar_arrive_expect_tx(bar0 + 8 * s, bytes);
      asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(buf0 + s * kBulkBytes), "l"(src), "r"(bytes), "r"(bar0 + 8 * s) : "memory");
    };
    // my tiles: blockIdx.x, blockIdx.x + gridDim.x, ...
    size_t next_load = blockIdx.x;
    uint32_t loaded = 0, done = 0;
    for (; loaded < kBulkStages && next_load < total_tiles; ++loaded, next_load += gridDim.x)
      issue_load(next_load, loaded % kBulkStages);
    bool ok = true;
    for (size_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++done) {
      const int s = done % kBulkStages;
      if (!(ok = mbar_wait(bar0 + 8 * s, (done / kBulkStages) & 1, wc, 50))) break;
      const float* src; float* dst; uint32_t bytes;
      tile_info(t, &src, &dst, &bytes);
      asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
                   ::"l"(dst), "r"(buf0 + s * kBulkBytes), "r"(bytes) : "memory");
      bulk_commit_group();
      if (next_load < total_tiles) {
        // the stage about to be refilled is the one just handed to the reduce: wait until it has been read
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        issue_load(next_load, s);
        ++loaded;
        next_load += gridDim.x;
      }
    }
    bulk_wait_group0();
    __threadfence_system();
  }
  finish_and_signal(ctrs, nranks, done_slot);
}

__global__ void wait_counter_kernel(const unsigned long long* ctr, unsigned long long expected,
                                    unsigned long long budget_ns, int* status) {
  if (threadIdx.x == 0 && blockIdx.x == 0) bounded_wait_ge(ctr, expected, budget_ns, status, /*detail=*/0);
}

// ---------------------------------------------------------------- one-sided count posting ---------------------
// `sync` without a host collective: every producer stores, on each owner, how many contributions it has sent to
// that owner so far (cumulative, low 32 bits) together with the number of the synchronisation it belongs to (high
// 32 bits), in the slot reserved for that producer.  The owner's wait kernel collects one posting of the current
// synchronisation from every producer, adds the counts up and then waits for its arrival counter to reach the
// sum.  Both waits are bounded and report through the status word.
__global__ void post_counts_kernel(const __grid_constant__ PostedCounts pc) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < pc.n)
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(pc.slot_addr[i]), "l"(pc.value[i]) : "memory");
}

__global__ void wait_posted_kernel(const unsigned long long* slots, int nprod, unsigned long long epoch,
                                   const unsigned long long* ctr, unsigned long long budget_ns, int* status,
                                   unsigned long long* expected_out) {
  const int lane = threadIdx.x;
  unsigned long long sum = 0;
  bool ok = true;
  const uint64_t t0 = globaltimer_ns();
  for (int p = lane; p < nprod && ok; p += 32) {
    unsigned long long v = ld_acquire_sys(slots + p);
    while ((v >> 32) < epoch) {
      __nanosleep(256);
      if (globaltimer_ns() - t0 > budget_ns) {
        report(status, kErrWaitTimeout, 1000 + p, static_cast<int>(v >> 32));  // producer p never posted
        ok = false;
        break;
      }
      v = ld_acquire_sys(slots + p);
    }
    sum += v & 0xffffffffull;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  ok = __all_sync(0xffffffffu, ok);
  if (lane == 0 && ok) {
    if (expected_out != nullptr) *expected_out = sum;
    const uint64_t spent = globaltimer_ns() - t0;
    bounded_wait_ge(ctr, sum, budget_ns > spent ? budget_ns - spent : 0, status, /*detail=*/0);
  }
}

int grid_for(size_t tiles, int sm_count) {
  // ODC_COMM_CTAS caps the grid of the communication kernels: fewer CTAs leave more of each SM to the GEMMs
  // they overlap with, at the price of fewer bytes in flight on the links
  static const int env_cap = [] {
    const char* e = getenv("ODC_COMM_CTAS");
    return e != nullptr ? atoi(e) : 0;
  }();
  size_t cap = env_cap > 0 ? size_t(env_cap) : size_t(sm_count) * 2;
  size_t g = tiles < cap ? tiles : cap;
  return g < 1 ? 1 : static_cast<int>(g);
}

}  // namespace

cudaError_t launch_gather(const long long* peers, void* out, size_t n, int src_elem_size, int dst_elem_size,
                          bool src_is_f32_dst_is_bf16, int nranks, int start, bool check, int* status,
                          int sm_count, cudaStream_t stream, size_t src_region_elems) {
  if (n == 0 || nranks == 0) return cudaSuccess;
  if (src_is_f32_dst_is_bf16) {
    const size_t tiles = ((n / 8 + kThreads * 2 - 1) / (kThreads * 2) + 1) * nranks;
    gather_f32_to_bf16_kernel<<<grid_for(tiles, sm_count), kThreads, 0, stream>>>(
        peers, static_cast<__nv_bfloat16*>(out), n, nranks, start, check ? 1 : 0, status, src_region_elems);
  } else {
    if (src_elem_size != dst_elem_size) return cudaErrorInvalidValue;
    const size_t row_bytes = n * src_elem_size;
    const int vec_ok = ((row_bytes % 16) == 0 || nranks == 1) && (reinterpret_cast<uintptr_t>(out) % 16) == 0;
    const size_t tiles = ((row_bytes / 16 + kTileVecs - 1) / kTileVecs + 1) * nranks;
    gather_copy_kernel<<<grid_for(tiles, sm_count), kThreads, 0, stream>>>(
        peers, static_cast<unsigned char*>(out), row_bytes, nranks, start, vec_ok, check ? 1 : 0, status,
        src_region_elems * src_elem_size);
  }
  return cudaGetLastError();
}

cudaError_t launch_scatter_accumulate(const void* inp, int in_kind, const long long* accs, int acc_kind,
                                      const long long* ctrs, size_t n, int nranks, int start, float scale,
                                      unsigned int* done_slot, int sm_count, cudaStream_t stream, int* status_for_bulk,
                                      long long acc_len) {
  if (nranks == 0) return cudaSuccess;
  const size_t tiles = ((n / 4 + kTileVecs - 1) / kTileVecs + 1) * nranks;
  const int grid = grid_for(tiles, sm_count);
  const int vec_ok = ((n % 4) == 0 || nranks == 1) && (reinterpret_cast<uintptr_t>(inp) % 16) == 0;
  static const bool bulk_enabled = [] {
    // opt-in: measured at 2 GPUs it does not beat the per-thread red.add kernel (426 vs 479 GB/s on 256 MiB
    // shards including the arrival wait), so the red.add kernel stays the default
    const char* e = getenv("ODC_SCATTER_BULK");
    return e != nullptr && e[0] == '1';
  }();
  if (bulk_enabled && acc_kind == kF32 && in_kind == kF32 && scale == 1.0f && (n % 4) == 0 && n * sizeof(float) >= 65536 &&
      (reinterpret_cast<uintptr_t>(inp) % 16) == 0) {
    static bool attr_set = false;
    if (!attr_set) {
      cudaError_t e = cudaFuncSetAttribute(scatter_acc_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBulkSmem);
      if (e != cudaSuccess) return e;
      attr_set = true;
    }
    const size_t bulk_tiles = ((n * sizeof(float) + kBulkBytes - 1) / kBulkBytes) * nranks;
    const int bulk_grid = bulk_tiles < size_t(sm_count) ? static_cast<int>(bulk_tiles) : sm_count;
    scatter_acc_bulk_kernel<<<bulk_grid, 32, kBulkSmem, stream>>>(static_cast<const float*>(inp), accs, ctrs, n, nranks,
                                                                start, done_slot, status_for_bulk, acc_len);
  } else if (acc_kind == kF32 && in_kind == kF32) {
    scatter_acc_f32_kernel<float><<<grid, kThreads, 0, stream>>>(static_cast<const float*>(inp), accs, ctrs, n,
                                                                 nranks, start, scale, done_slot, vec_ok, acc_len,
                                                                 status_for_bulk);
  } else if (acc_kind == kF32 && in_kind == kBF16) {
    scatter_acc_f32_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(inp), accs, ctrs, n, nranks, start, scale, done_slot, vec_ok, acc_len,
        status_for_bulk);
  } else if (acc_kind == kBF16 && in_kind == kBF16) {
    scatter_acc_bf16_kernel<<<grid, kThreads, 0, stream>>>(static_cast<const __nv_bfloat16*>(inp), accs, ctrs, n,
                                                          nranks, start, scale, done_slot, acc_len, status_for_bulk);
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_scatter_accumulate_segments(ScatterSegments segs, int in_kind, const long long* accs,
                                               const long long* ctrs, int nranks, int start, float scale,
                                               unsigned int* done_slot, int sm_count, cudaStream_t stream,
                                               long long acc_len, int* status) {
  if (nranks == 0) return cudaSuccess;
  if (segs.count < 0 || segs.count > kMaxScatterSegments) return cudaErrorInvalidValue;
  constexpr long long kTileElems = static_cast<long long>(kTileVecs) * 4;
  const int in_size = in_kind == kF32 ? 4 : 2;
  long long tiles = 0;
  for (int s = 0; s < segs.count; ++s) {
    if (segs.chunk[s] < 0 || segs.total[s] < 0 || segs.dst[s] < 0) return cudaErrorInvalidValue;
    segs.tile_prefix[s] = tiles;
    tiles += (segs.chunk[s] + kTileElems - 1) / kTileElems;
    // vector path: every owner's chunk starts on a 16-byte (fp32) / 8-byte (bf16) boundary of the source and on a
    // 16-byte boundary of the accumulator
    const bool src_ok = (reinterpret_cast<uintptr_t>(segs.src[s]) % (4 * in_size)) == 0 && (segs.chunk[s] % 4) == 0;
    segs.vec[s] = (src_ok && (segs.dst[s] % 4) == 0) ? 1 : 0;
  }
  segs.tile_prefix[segs.count] = tiles;
  const int grid = grid_for(static_cast<size_t>(tiles) * nranks + 1, sm_count);
  if (in_kind == kF32) {
    scatter_acc_segments_kernel<float><<<grid, kThreads, 0, stream>>>(segs, accs, ctrs, nranks, start, scale, done_slot,
                                                                      acc_len, status);
  } else if (in_kind == kBF16) {
    scatter_acc_segments_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(segs, accs, ctrs, nranks, start, scale,
                                                                            done_slot, acc_len, status);
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_post_counts(const PostedCounts& pc, cudaStream_t stream) {
  if (pc.n <= 0) return cudaSuccess;
  if (pc.n > kMaxPostedCounts) return cudaErrorInvalidValue;
  post_counts_kernel<<<(pc.n + 127) / 128, 128, 0, stream>>>(pc);
  return cudaGetLastError();
}

cudaError_t launch_wait_posted(const void* slots, int nprod, unsigned long long epoch, const void* ctr,
                               unsigned long long budget_ns, int* status, unsigned long long* expected_out,
                               cudaStream_t stream) {
  wait_posted_kernel<<<1, 32, 0, stream>>>(static_cast<const unsigned long long*>(slots), nprod, epoch,
                                           static_cast<const unsigned long long*>(ctr), budget_ns, status, expected_out);
  return cudaGetLastError();
}

cudaError_t launch_wait_counter(const void* ctr, unsigned long long expected, unsigned long long budget_ns,
                                int* status, cudaStream_t stream) {
  wait_counter_kernel<<<1, 32, 0, stream>>>(static_cast<const unsigned long long*>(ctr), expected, budget_ns,
                                            status);
  return cudaGetLastError();
}

}  // namespace odc
