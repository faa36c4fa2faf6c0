// Host-callable launchers of every kernel in this package.  Plain pointers + stream: no PyTorch
// headers, so kernel files compile in seconds; the binding layer converts tensors.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace odc {

enum DType : int { kF32 = 0, kBF16 = 1, kF16 = 2 };

// ---- communication -------------------------------------------------------------------------
// Debug launches (ODC_DEBUG_BOUNDS=1): `check` / a non-zero `src_region_elems` / `acc_len` make the kernel verify,
// before it touches anything, that the rotation start names a member of the group, that no table entry is null or
// misaligned, and that the elements it is about to read (gather) or add (scatter) fit the DECLARED length of the
// registered region.  A refused launch sets kErrBounds / kErrPeerIndex in the status word and returns normally.
cudaError_t launch_gather(const long long* peers, void* out, size_t n, int src_elem_size, int dst_elem_size,
                          bool src_is_f32_dst_is_bf16, int nranks, int start, bool check, int* status,
                          int sm_count, cudaStream_t stream, size_t src_region_elems = 0);
cudaError_t launch_scatter_accumulate(const void* inp, int in_kind, const long long* accs, int acc_kind,
                                      const long long* ctrs, size_t n, int nranks, int start, float scale,
                                      unsigned int* done_slot, int sm_count, cudaStream_t stream,
                                      int* status_for_bulk = nullptr, long long acc_len = 0);
// scatter_accumulate taken straight from up to kMaxScatterSegments contiguous gradient tensors (fp32 accumulators
// only).  The caller fills count/src/chunk/total/dst; the launcher derives tile_prefix and vec.
constexpr int kMaxScatterSegments = 32;
struct ScatterSegments {
  int count;
  const void* src[kMaxScatterSegments];       // contiguous gradient tensor
  long long chunk[kMaxScatterSegments];       // elements per owner (dim-0 chunk of the padded tensor)
  long long total[kMaxScatterSegments];       // elements that exist (owners past the end get fewer or none)
  long long dst[kMaxScatterSegments];         // element offset inside every owner's accumulator
  long long tile_prefix[kMaxScatterSegments + 1];
  int vec[kMaxScatterSegments];
};
cudaError_t launch_scatter_accumulate_segments(ScatterSegments segs, int in_kind, const long long* accs,
                                               const long long* ctrs, int nranks, int start, float scale,
                                               unsigned int* done_slot, int sm_count, cudaStream_t stream,
                                               long long acc_len = 0, int* status = nullptr);
cudaError_t launch_wait_counter(const void* ctr, unsigned long long expected, unsigned long long budget_ns,
                                int* status, cudaStream_t stream);
// One-sided exchange of the dispatch counts (what `sync` needs to know how many arrivals to wait for).
// post: value[i] = (synchronisation number << 32) | contributions sent so far to owner i, stored with a system-scope
// release at slot_addr[i] (this producer's slot on owner i).  wait: collect nprod postings of `epoch` from the
// local slots, then wait until the arrival counter reaches their sum; bounded, reports through `status`.
constexpr int kMaxPostedCounts = 72;
struct PostedCounts {
  int n;
  long long slot_addr[kMaxPostedCounts];
  unsigned long long value[kMaxPostedCounts];
};
cudaError_t launch_post_counts(const PostedCounts& pc, cudaStream_t stream);
cudaError_t launch_wait_posted(const void* slots, int nprod, unsigned long long epoch, const void* ctr,
                               unsigned long long budget_ns, int* status, unsigned long long* expected_out,
                               cudaStream_t stream);

// ---- single-primitive test kernels (device_prims.cu) ---------------------------------------------
cudaError_t launch_put_block(void* remote_dst, const void* local_src, size_t bytes, cudaStream_t s);
cudaError_t launch_get_block(void* local_dst, const void* remote_src, size_t bytes, cudaStream_t s);
cudaError_t launch_scalar_put_get(int* remote_word, int value, int* readback, cudaStream_t s);
cudaError_t launch_atomic_test(int* word, int* cas_seen, int* swap_seen, int ctas, int expected_old, int cas_new,
                               int swap_new, cudaStream_t s);
cudaError_t launch_grid_barrier_test(unsigned int* counter, int* slots, int* out, int ctas,
                                     unsigned long long budget_ns, int* status, cudaStream_t s);

// ---- elementwise / normalisation (bf16 activations, fp32 math) -----------------------------
cudaError_t launch_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int cols, float eps,
                               int sm_count, cudaStream_t stream);
// partial: [grid, cols] fp32 scratch (nullptr: in-kernel atomics into dw), dw: [cols] fp32; dres: optional bf16
// [rows, cols] gradient that reached x through a residual connection, added to dx in the same pass
cudaError_t launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                               float* partial, float* dw, int rows, int cols, int grid, cudaStream_t stream,
                               const void* dres = nullptr);
int rmsnorm_bwd_grid(int rows, int sm_count);
cudaError_t launch_rope_qkv(const void* in, void* out, const long long* pos, int tokens, int n_q, int n_kv,
                            int head_dim, float theta, bool inverse, cudaStream_t stream);
cudaError_t launch_swiglu_fwd(const void* gate_up, void* out, long long rows, int f, int sm_count,
                              cudaStream_t stream);
cudaError_t launch_swiglu_bwd(const void* dy, const void* gate_up, void* dgate_up, long long rows, int f,
                              int sm_count, cudaStream_t stream);
// logits [rows, vocab] bf16 are overwritten by scale * (softmax - onehot); loss += sum scale * nll
cudaError_t launch_ce_fwd_bwd(void* logits, const long long* labels, const float* loss_scale, float* loss,
                              int rows, int vocab, long long ignore_index, cudaStream_t stream);
// per_token[row] = log_softmax(logits[row])[labels[row]] (0 where the label is ignore_index); logits are only read
cudaError_t launch_token_logprobs(const void* logits, const long long* labels, float* per_token, int rows, int vocab,
                                  long long ignore_index, cudaStream_t stream);
cudaError_t launch_adamw(float* p, const void* g, int g_kind, float* m, float* v, void* p_lowp, size_t n, float lr,
                         float beta1, float beta2, float eps, float wd, float bc1, float bc2, float grad_scale,
                         int sm_count, cudaStream_t stream);
cudaError_t launch_cast_f32_to_bf16(const float* in, void* out, size_t n, int sm_count, cudaStream_t stream);
cudaError_t launch_sumsq(const void* x, int kind, size_t n, float* out, int sm_count, cudaStream_t stream);

// ---- tcgen05 GEMM ----------------------------------------------------------------------------
// layout: 0 = "nt" C[M,N] = A[M,K] B[N,K]^T ; 1 = "nn" C = A[M,K] B[K,N] ; 2 = "tn" C = A[K,M]^T B[K,N]
// All operands row-major bf16; C is bf16 or fp32; bias (bf16, length N) optional; accumulate adds into C.
struct GemmPlan;
cudaError_t gemm_bf16(const void* a, const void* b, void* c, int c_kind, const void* bias, int M, int N, int K,
                      int layout, bool accumulate, long long lda, long long ldb, long long ldc, int* status,
                      int sm_count, cudaStream_t stream, const void* residual = nullptr, long long ldr = 0,
                      int pair_mode = -1 /* -1: ODC_GEMM_PAIR decides, 0: single-CTA kernel, 1: CTA-pair kernel */);

// Same contract on CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles).  Returns cudaErrorNotSupported for shapes it
// does not take (M or N below 256, bf16 accumulation); gemm_bf16 tries it first unless ODC_GEMM_PAIR=0.
cudaError_t gemm_bf16_pair(const void* a, const void* b, void* c, int c_kind, const void* bias, int M, int N, int K,
                           int layout, bool accumulate, long long lda, long long ldb, long long ldc, int* status,
                           int sm_count, cudaStream_t stream, const void* residual = nullptr, long long ldr = 0);

cudaError_t gemm_wgrad_scatter_pair(const void* dy, const void* x, int tokens, int n_out, int k_in, long long ld_dy,
                                    long long ld_x, const long long* acc_addrs_host, const long long* ctr_ptrs,
                                    long long acc_offset, int rows_per_rank, int nranks, float scale,
                                    unsigned int* done_slot, int* status, int sm_count, cudaStream_t stream,
                                    int start_rank = 0);
cudaError_t gemm_gather_pair(bool dgrad, const void* a, const long long* shard_ptrs, void* w_local, void* out,
                             const void* bias, int M, int w_rows, int w_cols, long long lda, long long ldo,
                             int rows_per_rank, int nranks, unsigned int* group_flags, int* status, int sm_count,
                             cudaStream_t stream, const void* residual = nullptr, long long ldr = 0, int start_rank = 0);

// ---- GEMMs fused with the on-demand primitives ---------------------------------------------------
// dW[n_out, k_in] = dY[tokens, n_out]^T X[tokens, k_in]; row r of dW is added (x scale) into
// accumulator acc_ptrs[r / rows_per_rank] at element acc_offset + (r % rows_per_rank) * k_in.
cudaError_t gemm_wgrad_scatter(const void* dy, const void* x, int tokens, int n_out, int k_in, long long ld_dy,
                               long long ld_x, const long long* acc_ptrs, const long long* ctr_ptrs,
                               long long acc_offset, int rows_per_rank, int nranks, float scale,
                               unsigned int* done_slot, int* status, int sm_count, cudaStream_t stream);
// Same contract, but output boxes go through shared memory and TMA bulk reduce-add into the owners' accumulators.
// acc_addrs_host: HOST array of the accumulators' addresses (tensor maps are built on the host).  Returns
// cudaErrorNotSupported when rows_per_rank is not a multiple of 128 or there are more than 8 owners.
cudaError_t gemm_wgrad_scatter_tma(const void* dy, const void* x, int tokens, int n_out, int k_in, long long ld_dy,
                                   long long ld_x, const long long* acc_addrs_host, const long long* ctr_ptrs,
                                   long long acc_offset, int rows_per_rank, int nranks, float scale,
                                   unsigned int* done_slot, int* status, int sm_count, cudaStream_t stream,
                                   int start_rank = 0);
// Y[M, N] = X[M, K] W[N, K]^T with rank r holding rows [r * rows_per_rank, ...) of W at shard_ptrs[r];
// w_local [N, K] receives the gathered weight; panel_flags needs ceil(N / 256) words.
cudaError_t gemm_gather_nt(const void* x, const long long* shard_ptrs, void* w_local, void* y, const void* bias,
                           int M, int N, int K, long long ldx, long long ldy, int rows_per_rank, int nranks,
                           int start_rank, unsigned int* panel_flags, int* status, int sm_count,
                           cudaStream_t stream, const void* residual = nullptr, long long ldr = 0);
// dX[M, k_in] = dY[M, n_out] W[n_out, k_in] with W row-sharded as above: the gathered rows are the reduction
// dimension, so the k-loop of every output tile follows the arrival of the 256-row groups (first tile of a CTA)
// and later tiles find the whole weight in w_local.  group_flags needs ceil(n_out / 256) words.
cudaError_t gemm_gather_nn(const void* dy, const long long* shard_ptrs, void* w_local, void* dx, int M, int n_out,
                           int k_in, long long lddy, long long lddx, int rows_per_rank, int nranks,
                           unsigned int* group_flags, int* status, int sm_count, cudaStream_t stream,
                           int start_rank = 0);

// ---- varlen attention ------------------------------------------------------------------------
cudaError_t attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu_seqlens,
                     int num_seqs, int total_tokens, int max_seqlen, int n_q, int n_kv, int head_dim,
                     long long q_stride, long long kv_stride, long long o_stride, float scale, bool causal,
                     int* status, int sm_count, cudaStream_t stream);
cudaError_t attn_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o, const float* lse,
                     void* dq, void* dk, void* dv, float* delta, float* dq_acc, const int* cu_seqlens, int num_seqs,
                     int total_tokens, int max_seqlen, int n_q, int n_kv, int head_dim, long long q_stride,
                     long long kv_stride, long long o_stride, long long dq_stride, long long dkv_stride, float scale,
                     bool causal, int* status, int sm_count, cudaStream_t stream);

}  // namespace odc
