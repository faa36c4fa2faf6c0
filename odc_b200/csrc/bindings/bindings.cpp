// Python bindings: tensors in, raw pointers + current stream out to the launchers in kernels/api.h.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <mutex>
#include <unordered_map>

#include "../heap/symm_heap.h"
#include "../kernels/api.h"
#include "../kernels/tensor_map.h"

namespace py = pybind11;
using torch::Tensor;

namespace {

void check(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e));
}

int sm_count() {
  static int n = [] {
    int dev = 0, v = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
    return v > 0 ? v : 148;
  }();
  return n;
}

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

int kind_of(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return odc::kF32;
    case at::kBFloat16: return odc::kBF16;
    case at::kHalf: return odc::kF16;
    default: TORCH_CHECK(false, "unsupported dtype ", t);
  }
}

// Ring of self-resetting completion counters used by scatter_accumulate launches.  A slot is zero again once the
// last CTA of its launch has finished, so a slot may be handed out again only after that launch has run: with
// kDoneSlots slots this holds while fewer than kDoneSlots such launches are queued or running per device.  CUDA
// itself blocks the launching thread long before that many kernels are pending on a device (its launch queue holds
// on the order of a thousand), which is what bounds the number in flight.
constexpr unsigned long long kDoneSlots = 16384;
unsigned int* next_done_slot(int device) {
  static std::mutex mu;
  static std::unordered_map<int, Tensor> rings;
  static std::unordered_map<int, unsigned long long> seq;
  std::lock_guard<std::mutex> lock(mu);
  auto it = rings.find(device);
  if (it == rings.end()) {
    auto t = torch::zeros({static_cast<int64_t>(kDoneSlots)}, torch::dtype(torch::kInt32).device(torch::kCUDA, device));
    it = rings.emplace(device, t).first;
    seq[device] = 0;
  }
  unsigned long long s = seq[device]++;
  return reinterpret_cast<unsigned int*>(it->second.data_ptr<int>()) + (s % kDoneSlots);
}

// ---------------------------------------------------------------------------------------- heap
uintptr_t heap_create(int rank, int world, int device, size_t bytes, const std::string& mode,
                      const std::string& token) {
  return reinterpret_cast<uintptr_t>(odc::heap_create(rank, world, device, bytes, mode, token));
}
odc::Heap* H(uintptr_t h) { return reinterpret_cast<odc::Heap*>(h); }

Tensor tensor_from_ptr(uintptr_t ptr, int64_t numel, at::ScalarType dtype, int device) {
  auto opts = torch::TensorOptions().dtype(dtype).device(torch::kCUDA, device);
  return torch::from_blob(reinterpret_cast<void*>(ptr), {numel}, [](void*) {}, opts);
}

py::bytes get_ipc_handle(const Tensor& t) {
  TORCH_CHECK(t.is_cuda(), "get_ipc_handle expects a CUDA tensor");
  c10::cuda::CUDAGuard g(t.device());
  odc::bind_device(t.get_device());
  return py::bytes(odc::ipc_export(t.data_ptr()));
}

Tensor reconstruct_tensor(const std::string& blob, std::vector<int64_t> shape, at::ScalarType dtype) {
  void* p = odc::ipc_import(blob);
  int dev = 0;
  cudaGetDevice(&dev);
  auto opts = torch::TensorOptions().dtype(dtype).device(torch::kCUDA, dev);
  return torch::from_blob(p, shape, [](void*) {}, opts);
}

// ---------------------------------------------------------------------------------------- comm
void gather(Tensor out2d, Tensor table, int64_t n, at::ScalarType src_dtype, int my_index, bool checkb,
            Tensor status, int64_t src_region_elems) {
  c10::cuda::CUDAGuard g(out2d.device());
  odc::bind_device(out2d.get_device());
  const int nranks = static_cast<int>(table.numel());
  TORCH_CHECK(out2d.is_contiguous() && out2d.numel() == n * nranks, "gather: bad output shape");
  const int ssz = static_cast<int>(c10::elementSize(src_dtype));
  const int dsz = static_cast<int>(out2d.element_size());
  const bool narrow = (src_dtype == at::kFloat && out2d.scalar_type() == at::kBFloat16);
  TORCH_CHECK(narrow || src_dtype == out2d.scalar_type(), "gather: only same-dtype or fp32->bf16");
  check(odc::launch_gather(table.data_ptr<int64_t>() ? reinterpret_cast<const long long*>(table.data_ptr<int64_t>()) : nullptr,
                           out2d.data_ptr(), static_cast<size_t>(n), ssz, dsz, narrow, nranks, my_index, checkb,
                           status.data_ptr<int>(), sm_count(), cur_stream(),
                           checkb ? static_cast<size_t>(src_region_elems) : 0),
        "gather launch");
}

void scatter_accumulate(Tensor inp2d, Tensor acc_table, Tensor ctr_table, int64_t n, at::ScalarType acc_dtype,
                        int my_index, double scale, bool checkb, Tensor status, int64_t acc_region_elems) {
  c10::cuda::CUDAGuard g(inp2d.device());
  odc::bind_device(inp2d.get_device());
  const int nranks = static_cast<int>(acc_table.numel());
  TORCH_CHECK(inp2d.is_contiguous() && inp2d.numel() == n * nranks, "scatter_accumulate: bad input shape");
  check(odc::launch_scatter_accumulate(inp2d.data_ptr(), kind_of(inp2d.scalar_type()),
                                       reinterpret_cast<const long long*>(acc_table.data_ptr<int64_t>()),
                                       kind_of(acc_dtype),
                                       reinterpret_cast<const long long*>(ctr_table.data_ptr<int64_t>()),
                                       static_cast<size_t>(n), nranks, my_index, static_cast<float>(scale),
                                       next_done_slot(inp2d.get_device()), sm_count(), cur_stream(),
                                       status.data_ptr<int>(), checkb ? acc_region_elems : 0),
        "scatter_accumulate launch");
}

bool scatter_accumulate_segments(std::vector<Tensor> grads, std::vector<int64_t> chunk_numels,
                                 std::vector<int64_t> dst_offsets, Tensor acc_table, Tensor ctr_table,
                                 at::ScalarType acc_dtype, int my_index, double scale, bool checkb,
                                 c10::optional<Tensor> status, int64_t acc_region_elems) {
  // Returns false (nothing launched) when the list does not fit this path; the caller then flattens the gradients.
  if (grads.empty() || grads.size() > static_cast<size_t>(odc::kMaxScatterSegments) || acc_dtype != at::kFloat) return false;
  TORCH_CHECK(grads.size() == chunk_numels.size() && grads.size() == dst_offsets.size(),
              "scatter_accumulate_segments: one chunk size and one offset per gradient");
  const auto dt = grads[0].scalar_type();
  if (dt != at::kFloat && dt != at::kBFloat16) return false;
  odc::ScatterSegments segs{};
  segs.count = static_cast<int>(grads.size());
  for (size_t i = 0; i < grads.size(); ++i) {
    const Tensor& g = grads[i];
    if (!g.is_cuda() || !g.is_contiguous() || g.scalar_type() != dt || g.device() != grads[0].device()) return false;
    segs.src[i] = g.data_ptr();
    segs.chunk[i] = chunk_numels[i];
    segs.total[i] = g.numel();
    segs.dst[i] = dst_offsets[i];
  }
  c10::cuda::CUDAGuard guard(grads[0].device());
  odc::bind_device(grads[0].get_device());
  const int nranks = static_cast<int>(acc_table.numel());
  check(odc::launch_scatter_accumulate_segments(segs, kind_of(dt),
                                                reinterpret_cast<const long long*>(acc_table.data_ptr<int64_t>()),
                                                reinterpret_cast<const long long*>(ctr_table.data_ptr<int64_t>()), nranks,
                                                my_index, static_cast<float>(scale),
                                                next_done_slot(grads[0].get_device()), sm_count(), cur_stream(),
                                                (checkb && status.has_value()) ? acc_region_elems : 0,
                                                status.has_value() ? status->data_ptr<int>() : nullptr),
        "scatter_accumulate_segments launch");
  return true;
}

void wait_counter(Tensor counter, int64_t expected, int64_t timeout_ms, Tensor status) {
  c10::cuda::CUDAGuard g(counter.device());
  odc::bind_device(counter.get_device());
  check(odc::launch_wait_counter(counter.data_ptr(), static_cast<unsigned long long>(expected),
                                 static_cast<unsigned long long>(timeout_ms) * 1000000ull, status.data_ptr<int>(),
                                 cur_stream()),
        "wait_counter launch");
}

void post_counts(std::vector<int64_t> slot_addrs, std::vector<int64_t> counts, int64_t epoch, int device) {
  c10::cuda::CUDAGuard g(c10::Device(c10::kCUDA, static_cast<c10::DeviceIndex>(device)));
  odc::bind_device(device);
  TORCH_CHECK(slot_addrs.size() == counts.size() && slot_addrs.size() <= size_t(odc::kMaxPostedCounts),
              "post_counts: at most ", odc::kMaxPostedCounts, " owners");
  odc::PostedCounts pc{};
  pc.n = static_cast<int>(slot_addrs.size());
  for (int i = 0; i < pc.n; ++i) {
    TORCH_CHECK(slot_addrs[i] != 0 && (slot_addrs[i] & 7) == 0, "post_counts: bad slot address");
    TORCH_CHECK(counts[i] >= 0 && counts[i] < (int64_t(1) << 32), "post_counts: count out of range");
    pc.slot_addr[i] = slot_addrs[i];
    pc.value[i] = (static_cast<unsigned long long>(epoch) << 32) | static_cast<unsigned long long>(counts[i]);
  }
  check(odc::launch_post_counts(pc, cur_stream()), "post_counts launch");
}

void wait_posted(Tensor slots, int64_t nprod, int64_t epoch, Tensor counter, int64_t timeout_ms, Tensor status,
                 Tensor expected_out) {
  c10::cuda::CUDAGuard g(counter.device());
  odc::bind_device(counter.get_device());
  TORCH_CHECK(slots.scalar_type() == at::kLong && slots.numel() >= nprod && expected_out.scalar_type() == at::kLong,
              "wait_posted: int64 slots (one per producer) and an int64 output word");
  check(odc::launch_wait_posted(slots.data_ptr(), static_cast<int>(nprod), static_cast<unsigned long long>(epoch),
                                counter.data_ptr(), static_cast<unsigned long long>(timeout_ms) * 1000000ull,
                                status.data_ptr<int>(), reinterpret_cast<unsigned long long*>(expected_out.data_ptr()),
                                cur_stream()),
        "wait_posted launch");
}

// ---------------------------------------------------------------------------------------- ops
std::tuple<Tensor, Tensor> rmsnorm_fwd(Tensor x, Tensor w, double eps) {
  c10::cuda::CUDAGuard g(x.device());
  odc::bind_device(x.get_device());
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && x.scalar_type() == at::kBFloat16, "rmsnorm: x must be [T,H] bf16");
  TORCH_CHECK(w.scalar_type() == at::kBFloat16 && w.is_contiguous(), "rmsnorm: weight must be bf16");
  auto y = torch::empty_like(x);
  auto rstd = torch::empty({x.size(0)}, x.options().dtype(at::kFloat));
  check(odc::launch_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(),
                                static_cast<int>(x.size(0)), static_cast<int>(x.size(1)), static_cast<float>(eps),
                                sm_count(), cur_stream()),
        "rmsnorm_fwd");
  return {y, rstd};
}

std::tuple<Tensor, Tensor> rmsnorm_bwd(Tensor dy, Tensor x, Tensor w, Tensor rstd, bool fixed_order,
                                       c10::optional<Tensor> dres) {
  c10::cuda::CUDAGuard g(x.device());
  odc::bind_device(x.get_device());
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous() && dy.sizes() == x.sizes(), "rmsnorm_bwd: contiguous dy, x [T,H]");
  const int rows = static_cast<int>(x.size(0)), cols = static_cast<int>(x.size(1));
  auto dx = torch::empty_like(x);
  const int grid = odc::rmsnorm_bwd_grid(rows, sm_count());
  auto dw = torch::empty({cols}, x.options().dtype(at::kFloat));
  Tensor partial;
  float* partial_ptr = nullptr;
  if (fixed_order) {  // per-CTA column sums added up in a fixed order by a second pass (bitwise reproducible)
    partial = torch::empty({grid, cols}, x.options().dtype(at::kFloat));
    partial_ptr = partial.data_ptr<float>();
  }
  const void* dres_ptr = nullptr;
  if (dres.has_value()) {
    TORCH_CHECK(dres->is_contiguous() && dres->sizes() == x.sizes() && dres->scalar_type() == at::kBFloat16,
                "rmsnorm_bwd: residual gradient must be contiguous bf16 of x's shape");
    dres_ptr = dres->data_ptr();
  }
  check(odc::launch_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(),
                                partial_ptr, dw.data_ptr<float>(), rows, cols, grid, cur_stream(), dres_ptr),
        "rmsnorm_bwd");
  return {dx, dw};
}

Tensor rope_qkv(Tensor qkv, Tensor pos, int n_q, int n_kv, int head_dim, double theta, bool inverse) {
  c10::cuda::CUDAGuard g(qkv.device());
  odc::bind_device(qkv.get_device());
  TORCH_CHECK(qkv.dim() == 2 && qkv.is_contiguous() && qkv.scalar_type() == at::kBFloat16, "rope: qkv [T,W] bf16");
  TORCH_CHECK(qkv.size(1) == int64_t(n_q + 2 * n_kv) * head_dim, "rope: width mismatch");
  TORCH_CHECK(pos.scalar_type() == at::kLong && pos.numel() == qkv.size(0), "rope: position_ids int64 [T]");
  auto out = torch::empty_like(qkv);
  check(odc::launch_rope_qkv(qkv.data_ptr(), out.data_ptr(), reinterpret_cast<const long long*>(pos.data_ptr<int64_t>()),
                             static_cast<int>(qkv.size(0)), n_q, n_kv, head_dim, static_cast<float>(theta), inverse,
                             cur_stream()),
        "rope_qkv");
  return out;
}

Tensor swiglu_fwd(Tensor gu) {
  c10::cuda::CUDAGuard g(gu.device());
  odc::bind_device(gu.get_device());
  TORCH_CHECK(gu.is_contiguous() && gu.scalar_type() == at::kBFloat16, "swiglu: bf16 contiguous");
  const int f = static_cast<int>(gu.size(-1) / 2);
  auto sizes = gu.sizes().vec();
  sizes.back() = f;
  auto out = torch::empty(sizes, gu.options());
  check(odc::launch_swiglu_fwd(gu.data_ptr(), out.data_ptr(), gu.numel() / (2 * f), f, sm_count(), cur_stream()),
        "swiglu_fwd");
  return out;
}

Tensor swiglu_bwd(Tensor dy, Tensor gu) {
  c10::cuda::CUDAGuard g(gu.device());
  odc::bind_device(gu.get_device());
  const int f = static_cast<int>(gu.size(-1) / 2);
  auto out = torch::empty_like(gu);
  check(odc::launch_swiglu_bwd(dy.data_ptr(), gu.data_ptr(), out.data_ptr(), gu.numel() / (2 * f), f, sm_count(),
                               cur_stream()),
        "swiglu_bwd");
  return out;
}

void ce_fwd_bwd(Tensor logits, Tensor labels, c10::optional<Tensor> loss_scale, Tensor loss, int64_t ignore_index) {
  c10::cuda::CUDAGuard g(logits.device());
  odc::bind_device(logits.get_device());
  TORCH_CHECK(logits.dim() == 2 && logits.is_contiguous() && logits.scalar_type() == at::kBFloat16, "ce: logits bf16");
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.is_contiguous(), "ce: labels int64");
  const float* ls = nullptr;
  if (loss_scale.has_value()) {
    TORCH_CHECK(loss_scale->scalar_type() == at::kFloat && loss_scale->is_contiguous(), "ce: loss_scale fp32");
    ls = loss_scale->data_ptr<float>();
  }
  check(odc::launch_ce_fwd_bwd(logits.data_ptr(), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()), ls,
                               loss.data_ptr<float>(), static_cast<int>(logits.size(0)),
                               static_cast<int>(logits.size(1)), ignore_index, cur_stream()),
        "ce_fwd_bwd");
}

void token_logprobs(Tensor logits, Tensor labels, Tensor out, int64_t ignore_index) {
  c10::cuda::CUDAGuard g(logits.device());
  odc::bind_device(logits.get_device());
  TORCH_CHECK(logits.dim() == 2 && logits.is_contiguous() && logits.scalar_type() == at::kBFloat16, "token_logprobs: logits bf16");
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.is_contiguous() && labels.numel() == logits.size(0),
              "token_logprobs: one int64 label per row");
  TORCH_CHECK(out.scalar_type() == at::kFloat && out.is_contiguous() && out.numel() == logits.size(0) && out.is_cuda(),
              "token_logprobs: one fp32 output per row");
  check(odc::launch_token_logprobs(logits.data_ptr(), reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                                   out.data_ptr<float>(), static_cast<int>(logits.size(0)),
                                   static_cast<int>(logits.size(1)), ignore_index, cur_stream()),
        "token_logprobs");
}

void adamw_step(Tensor p, Tensor g, Tensor m, Tensor v, c10::optional<Tensor> p_lowp, double lr, double beta1,
                double beta2, double eps, double wd, int64_t step, double grad_scale) {
  c10::cuda::CUDAGuard guard(p.device());
  odc::bind_device(p.get_device());
  TORCH_CHECK(p.scalar_type() == at::kFloat && m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat,
              "adamw: fp32 master state");
  TORCH_CHECK(p.is_contiguous() && g.is_contiguous() && m.is_contiguous() && v.is_contiguous(), "adamw: contiguous");
  void* lp = nullptr;
  if (p_lowp.has_value()) {
    TORCH_CHECK(p_lowp->scalar_type() == at::kBFloat16 && p_lowp->numel() == p.numel(), "adamw: bf16 replica");
    lp = p_lowp->data_ptr();
  }
  const float bc1 = 1.f - std::pow(static_cast<float>(beta1), static_cast<float>(step));
  const float bc2 = 1.f - std::pow(static_cast<float>(beta2), static_cast<float>(step));
  check(odc::launch_adamw(p.data_ptr<float>(), g.data_ptr(), kind_of(g.scalar_type()), m.data_ptr<float>(),
                          v.data_ptr<float>(), lp, static_cast<size_t>(p.numel()), static_cast<float>(lr),
                          static_cast<float>(beta1), static_cast<float>(beta2), static_cast<float>(eps),
                          static_cast<float>(wd), bc1, bc2, static_cast<float>(grad_scale), sm_count(), cur_stream()),
        "adamw");
}

void cast_f32_to_bf16(Tensor in, Tensor out) {
  c10::cuda::CUDAGuard g(in.device());
  odc::bind_device(in.get_device());
  TORCH_CHECK(in.scalar_type() == at::kFloat && out.scalar_type() == at::kBFloat16 && in.numel() == out.numel() &&
                  in.is_contiguous() && out.is_contiguous(), "cast: fp32 -> bf16, same numel, contiguous");
  check(odc::launch_cast_f32_to_bf16(in.data_ptr<float>(), out.data_ptr(), static_cast<size_t>(in.numel()), sm_count(),
                                     cur_stream()),
        "cast");
}

void sumsq(Tensor x, Tensor out) {
  c10::cuda::CUDAGuard g(x.device());
  odc::bind_device(x.get_device());
  TORCH_CHECK(x.is_contiguous() && out.scalar_type() == at::kFloat, "sumsq: contiguous input, fp32 output");
  check(odc::launch_sumsq(x.data_ptr(), kind_of(x.scalar_type()), static_cast<size_t>(x.numel()), out.data_ptr<float>(),
                          sm_count(), cur_stream()),
        "sumsq");
}

Tensor& gemm_status(int device) {
  static std::mutex mu;
  static std::unordered_map<int, Tensor> st;
  std::lock_guard<std::mutex> lock(mu);
  auto it = st.find(device);
  if (it == st.end()) it = st.emplace(device, torch::zeros({4}, torch::dtype(torch::kInt32).device(torch::kCUDA, device))).first;
  return it->second;
}

Tensor kernel_status() {
  int dev = 0;
  cudaGetDevice(&dev);
  return gemm_status(dev);
}

void gemm(Tensor a, Tensor b, Tensor c, const std::string& layout, c10::optional<Tensor> bias, bool accumulate,
          c10::optional<Tensor> residual, int pair) {
  c10::cuda::CUDAGuard g(a.device());
  odc::bind_device(a.get_device());
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && c.dim() == 2, "gemm: 2-D operands");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16, "gemm: bf16 inputs");
  TORCH_CHECK(a.stride(1) == 1 && b.stride(1) == 1 && c.stride(1) == 1, "gemm: innermost stride must be 1");
  int lay, M, N, K;
  if (layout == "nt") {
    lay = 0; M = a.size(0); K = a.size(1); N = b.size(0);
    TORCH_CHECK(b.size(1) == K, "gemm nt: K mismatch");
  } else if (layout == "nn") {
    lay = 1; M = a.size(0); K = a.size(1); N = b.size(1);
    TORCH_CHECK(b.size(0) == K, "gemm nn: K mismatch");
  } else if (layout == "tn") {
    lay = 2; K = a.size(0); M = a.size(1); N = b.size(1);
    TORCH_CHECK(b.size(0) == K, "gemm tn: K mismatch");
  } else {
    TORCH_CHECK(false, "gemm: unknown layout ", layout);
  }
  TORCH_CHECK(c.size(0) == M && c.size(1) == N, "gemm: output shape mismatch");
  const void* bias_ptr = nullptr;
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == N && bias->is_contiguous(), "gemm: bias bf16 [N]");
    bias_ptr = bias->data_ptr();
  }
  const void* res_ptr = nullptr;
  long long ldr = 0;
  if (residual.has_value()) {
    TORCH_CHECK(residual->scalar_type() == at::kBFloat16 && residual->dim() == 2 && residual->size(0) == M &&
                    residual->size(1) == N && residual->stride(1) == 1, "gemm: residual bf16 [M,N]");
    res_ptr = residual->data_ptr();
    ldr = residual->stride(0);
  }
  cudaError_t e = odc::gemm_bf16(a.data_ptr(), b.data_ptr(), c.data_ptr(), kind_of(c.scalar_type()), bias_ptr, M, N, K,
                                 lay, accumulate, a.stride(0), b.stride(0), c.stride(0),
                                 gemm_status(a.get_device()).data_ptr<int>(), sm_count(), cur_stream(), res_ptr, ldr,
                                 pair);
  TORCH_CHECK(e == cudaSuccess, "gemm(", layout, ") M=", M, " N=", N, " K=", K, " lda=", a.stride(0), " ldb=", b.stride(0),
              " ldc=", c.stride(0), " align(a,b,c)=", reinterpret_cast<uintptr_t>(a.data_ptr()) % 16, ",",
              reinterpret_cast<uintptr_t>(b.data_ptr()) % 16, ",", reinterpret_cast<uintptr_t>(c.data_ptr()) % 16, ": ",
              cudaGetErrorString(e));
}

void gemm_wgrad_scatter(Tensor dy, Tensor x, Tensor acc_table, Tensor ctr_table, int64_t acc_offset,
                        int64_t rows_per_rank, double scale) {
  c10::cuda::CUDAGuard g(dy.device());
  odc::bind_device(dy.get_device());
  TORCH_CHECK(dy.dim() == 2 && x.dim() == 2 && dy.size(0) == x.size(0), "wgrad_scatter: dy [T,N], x [T,K]");
  TORCH_CHECK(dy.scalar_type() == at::kBFloat16 && x.scalar_type() == at::kBFloat16, "wgrad_scatter: bf16 inputs");
  TORCH_CHECK(dy.stride(1) == 1 && x.stride(1) == 1, "wgrad_scatter: innermost stride must be 1");
  check(odc::gemm_wgrad_scatter(dy.data_ptr(), x.data_ptr(), dy.size(0), dy.size(1), x.size(1), dy.stride(0),
                                x.stride(0), reinterpret_cast<const long long*>(acc_table.data_ptr<int64_t>()),
                                reinterpret_cast<const long long*>(ctr_table.data_ptr<int64_t>()), acc_offset,
                                static_cast<int>(rows_per_rank), static_cast<int>(acc_table.numel()),
                                static_cast<float>(scale), next_done_slot(dy.get_device()),
                                gemm_status(dy.get_device()).data_ptr<int>(), sm_count(), cur_stream()),
        "gemm_wgrad_scatter");
}

bool gemm_wgrad_scatter_tma(Tensor dy, Tensor x, std::vector<int64_t> acc_addrs, Tensor ctr_table, int64_t acc_offset,
                            int64_t rows_per_rank, double scale, int start_rank) {
  c10::cuda::CUDAGuard g(dy.device());
  odc::bind_device(dy.get_device());
  TORCH_CHECK(dy.dim() == 2 && x.dim() == 2 && dy.size(0) == x.size(0), "wgrad_scatter: dy [T,N], x [T,K]");
  TORCH_CHECK(dy.scalar_type() == at::kBFloat16 && x.scalar_type() == at::kBFloat16, "wgrad_scatter: bf16 inputs");
  TORCH_CHECK(dy.stride(1) == 1 && x.stride(1) == 1, "wgrad_scatter: innermost stride must be 1");
  std::vector<long long> addrs(acc_addrs.begin(), acc_addrs.end());
  cudaError_t e = odc::gemm_wgrad_scatter_tma(
      dy.data_ptr(), x.data_ptr(), dy.size(0), dy.size(1), x.size(1), dy.stride(0), x.stride(0), addrs.data(),
      reinterpret_cast<const long long*>(ctr_table.data_ptr<int64_t>()), acc_offset, static_cast<int>(rows_per_rank),
      static_cast<int>(addrs.size()), static_cast<float>(scale), next_done_slot(dy.get_device()),
      gemm_status(dy.get_device()).data_ptr<int>(), sm_count(), cur_stream(), start_rank);
  if (e == cudaErrorNotSupported) return false;  // shape not eligible: the caller uses the red.add variant
  check(e, "gemm_wgrad_scatter_tma");
  return true;
}

Tensor gemm_gather(Tensor x, Tensor shard_table, Tensor w_local, c10::optional<Tensor> bias, int64_t rows_per_rank,
                   int start_rank, c10::optional<Tensor> residual) {
  c10::cuda::CUDAGuard g(x.device());
  odc::bind_device(x.get_device());
  TORCH_CHECK(x.dim() == 2 && w_local.dim() == 2 && x.size(1) == w_local.size(1), "gemm_gather: x [M,K], w_local [N,K]");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && w_local.scalar_type() == at::kBFloat16 && w_local.is_contiguous() &&
                  x.stride(1) == 1, "gemm_gather: bf16, contiguous weight buffer");
  const int M = x.size(0), K = x.size(1), N = w_local.size(0);
  auto y = torch::empty({M, N}, x.options());
  auto flags = torch::empty({(N + 255) / 256}, x.options().dtype(at::kInt));
  const void* bias_ptr = nullptr;
  if (bias.has_value()) {
    TORCH_CHECK(bias->scalar_type() == at::kBFloat16 && bias->numel() == N, "gemm_gather: bias bf16 [N]");
    bias_ptr = bias->data_ptr();
  }
  const void* res_ptr = nullptr;
  long long ldr = 0;
  if (residual.has_value()) {
    TORCH_CHECK(residual->scalar_type() == at::kBFloat16 && residual->dim() == 2 && residual->size(0) == M &&
                    residual->size(1) == N && residual->stride(1) == 1, "gemm_gather: residual bf16 [M,N]");
    res_ptr = residual->data_ptr();
    ldr = residual->stride(0);
  }
  check(odc::gemm_gather_nt(x.data_ptr(), reinterpret_cast<const long long*>(shard_table.data_ptr<int64_t>()),
                            w_local.data_ptr(), y.data_ptr(), bias_ptr, M, N, K, x.stride(0), y.stride(0),
                            static_cast<int>(rows_per_rank), static_cast<int>(shard_table.numel()), start_rank,
                            reinterpret_cast<unsigned int*>(flags.data_ptr<int>()),
                            gemm_status(x.get_device()).data_ptr<int>(), sm_count(), cur_stream(), res_ptr, ldr),
        "gemm_gather");
  return y;
}

Tensor gemm_gather_dgrad(Tensor dy, Tensor shard_table, Tensor w_local, int64_t rows_per_rank, int start_rank) {
  c10::cuda::CUDAGuard g(dy.device());
  odc::bind_device(dy.get_device());
  TORCH_CHECK(dy.dim() == 2 && w_local.dim() == 2 && dy.size(1) == w_local.size(0),
              "gemm_gather_dgrad: dy [M,N], w_local [N,K]");
  TORCH_CHECK(dy.scalar_type() == at::kBFloat16 && w_local.scalar_type() == at::kBFloat16 && w_local.is_contiguous() &&
                  dy.stride(1) == 1, "gemm_gather_dgrad: bf16, contiguous weight buffer");
  const int M = dy.size(0), N = dy.size(1), K = w_local.size(1);
  auto dx = torch::empty({M, K}, dy.options());
  auto flags = torch::empty({(N + 255) / 256}, dy.options().dtype(at::kInt));
  check(odc::gemm_gather_nn(dy.data_ptr(), reinterpret_cast<const long long*>(shard_table.data_ptr<int64_t>()),
                            w_local.data_ptr(), dx.data_ptr(), M, N, K, dy.stride(0), dx.stride(0),
                            static_cast<int>(rows_per_rank), static_cast<int>(shard_table.numel()),
                            reinterpret_cast<unsigned int*>(flags.data_ptr<int>()),
                            gemm_status(dy.get_device()).data_ptr<int>(), sm_count(), cur_stream(), start_rank),
        "gemm_gather_dgrad");
  return dx;
}

std::tuple<Tensor, Tensor> attn_fwd(Tensor q, Tensor k, Tensor v, Tensor cu_seqlens, int max_seqlen, bool causal,
                                    double scale) {
  c10::cuda::CUDAGuard g(q.device());
  odc::bind_device(q.get_device());
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3, "attention: q/k/v are [T, H, D]");
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16,
              "attention: bf16 inputs");
  const int T = q.size(0), hq = q.size(1), d = q.size(2), hkv = k.size(1);
  TORCH_CHECK(q.stride(2) == 1 && q.stride(1) == d && k.stride(2) == 1 && k.stride(1) == d && v.stride(2) == 1 &&
                  v.stride(1) == d, "attention: heads must be packed within a token");
  TORCH_CHECK(k.stride(0) == v.stride(0), "attention: k and v must share a row stride");
  TORCH_CHECK(cu_seqlens.scalar_type() == at::kInt && cu_seqlens.is_contiguous(), "attention: cu_seqlens int32");
  auto o = torch::empty({T, hq, d}, q.options());
  auto lse = torch::empty({hq, T}, q.options().dtype(at::kFloat));
  check(odc::attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(),
                      cu_seqlens.data_ptr<int>(), static_cast<int>(cu_seqlens.numel() - 1), T, max_seqlen, hq, hkv, d,
                      q.stride(0), k.stride(0), o.stride(0), static_cast<float>(scale), causal,
                      gemm_status(q.get_device()).data_ptr<int>(), sm_count(), cur_stream()),
        "attn_fwd");
  return {o, lse};
}

std::tuple<Tensor, Tensor, Tensor, Tensor> attn_bwd(Tensor dout, Tensor q, Tensor k, Tensor v, Tensor o, Tensor lse,
                                                    Tensor cu_seqlens, int max_seqlen, bool causal, double scale,
                                                    bool fused_qkv) {
  c10::cuda::CUDAGuard g(q.device());
  odc::bind_device(q.get_device());
  const int T = q.size(0), hq = q.size(1), d = q.size(2), hkv = k.size(1);
  TORCH_CHECK(dout.is_contiguous() && dout.scalar_type() == at::kBFloat16, "attention bwd: dout contiguous bf16");
  TORCH_CHECK(o.stride(2) == 1 && o.stride(1) == d, "attention bwd: o heads packed");
  TORCH_CHECK(q.stride(2) == 1 && q.stride(1) == d && k.stride(2) == 1 && k.stride(1) == d && v.stride(2) == 1 &&
                  v.stride(1) == d && k.stride(0) == v.stride(0), "attention bwd: q/k/v layout");
  Tensor dq, dk, dv, dqkv;
  if (fused_qkv) {
    // one [T, (hq + 2 hkv) d] gradient; dq/dk/dv are column views of it, so slicing costs nothing in autograd
    dqkv = torch::empty({T, int64_t(hq + 2 * hkv) * d}, q.options());
    dq = dqkv.narrow(1, 0, int64_t(hq) * d).view({T, hq, d});
    dk = dqkv.narrow(1, int64_t(hq) * d, int64_t(hkv) * d).view({T, hkv, d});
    dv = dqkv.narrow(1, int64_t(hq + hkv) * d, int64_t(hkv) * d).view({T, hkv, d});
  } else {
    dq = torch::empty({T, hq, d}, q.options());
    dk = torch::empty({T, hkv, d}, q.options());
    dv = torch::empty({T, hkv, d}, q.options());
  }
  auto delta = torch::empty({hq, T}, q.options().dtype(at::kFloat));
  auto dq_acc = torch::empty({T, hq, d}, q.options().dtype(at::kFloat));
  check(odc::attn_bwd(dout.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr<float>(),
                      dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), delta.data_ptr<float>(), dq_acc.data_ptr<float>(),
                      cu_seqlens.data_ptr<int>(), static_cast<int>(cu_seqlens.numel() - 1), T, max_seqlen, hq, hkv, d,
                      q.stride(0), k.stride(0), o.stride(0), dq.stride(0), dk.stride(0), static_cast<float>(scale),
                      causal, gemm_status(q.get_device()).data_ptr<int>(), sm_count(), cur_stream()),
        "attn_bwd");
  return {dq, dk, dv, fused_qkv ? dqkv : dq};  // 4th: the fused gradient when requested
}

// --- single-primitive test entry points: addresses are plain integers so peers' mappings can be passed
void put_block(uintptr_t remote_dst, Tensor local_src) {
  c10::cuda::CUDAGuard g(local_src.device());
  odc::bind_device(local_src.get_device());
  check(odc::launch_put_block(reinterpret_cast<void*>(remote_dst), local_src.data_ptr(), local_src.nbytes(), cur_stream()),
        "put_block");
}
void get_block(Tensor local_dst, uintptr_t remote_src) {
  c10::cuda::CUDAGuard g(local_dst.device());
  odc::bind_device(local_dst.get_device());
  check(odc::launch_get_block(local_dst.data_ptr(), reinterpret_cast<const void*>(remote_src), local_dst.nbytes(),
                              cur_stream()), "get_block");
}
void scalar_put_get(uintptr_t remote_word, int value, Tensor readback) {
  c10::cuda::CUDAGuard g(readback.device());
  odc::bind_device(readback.get_device());
  check(odc::launch_scalar_put_get(reinterpret_cast<int*>(remote_word), value, readback.data_ptr<int>(), cur_stream()),
        "scalar_put_get");
}
void atomic_test(Tensor word, Tensor cas_seen, Tensor swap_seen, int expected_old, int cas_new, int swap_new) {
  c10::cuda::CUDAGuard g(word.device());
  odc::bind_device(word.get_device());
  check(odc::launch_atomic_test(word.data_ptr<int>(), cas_seen.data_ptr<int>(), swap_seen.data_ptr<int>(),
                                static_cast<int>(cas_seen.numel()), expected_old, cas_new, swap_new, cur_stream()),
        "atomic_test");
}
void grid_barrier_test(Tensor counter, Tensor slots, Tensor out, int64_t timeout_ms, Tensor status) {
  c10::cuda::CUDAGuard g(out.device());
  odc::bind_device(out.get_device());
  TORCH_CHECK(out.numel() <= sm_count(), "grid barrier needs co-resident CTAs: at most one per SM");
  check(odc::launch_grid_barrier_test(reinterpret_cast<unsigned int*>(counter.data_ptr<int>()), slots.data_ptr<int>(),
                                      out.data_ptr<int>(), static_cast<int>(out.numel()),
                                      static_cast<unsigned long long>(timeout_ms) * 1000000ull, status.data_ptr<int>(),
                                      cur_stream()), "grid_barrier_test");
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("heap_create", &heap_create);
  m.def("heap_grow", [](uintptr_t h, size_t n) { odc::heap_grow(H(h), n); }, py::call_guard<py::gil_scoped_release>());
  m.def("heap_ipc_handle", [](uintptr_t h) { return py::bytes(odc::heap_ipc_handle(H(h))); });
  m.def("heap_ipc_open", [](uintptr_t h, int r, const std::string& b) { odc::heap_ipc_open(H(h), r, b); });
  m.def("heap_base", [](uintptr_t h, int r) { return odc::heap_base(H(h), r); });
  m.def("heap_mapped", [](uintptr_t h) { return odc::heap_mapped(H(h)); });
  m.def("heap_destroy", [](uintptr_t h) { odc::heap_destroy(H(h)); });
  m.def("tensor_from_ptr", &tensor_from_ptr);
  m.def("get_ipc_handle", &get_ipc_handle);
  m.def("reconstruct_tensor", &reconstruct_tensor);
  // the trailing *_region_elems arguments are the DECLARED lengths the debug checks (check = true) hold the launch to
  m.def("gather", &gather, py::arg("out2d"), py::arg("table"), py::arg("n"), py::arg("src_dtype"), py::arg("my_index"),
        py::arg("check"), py::arg("status"), py::arg("src_region_elems") = 0);
  m.def("scatter_accumulate", &scatter_accumulate, py::arg("inp2d"), py::arg("acc_table"), py::arg("ctr_table"),
        py::arg("n"), py::arg("acc_dtype"), py::arg("my_index"), py::arg("scale"), py::arg("check"), py::arg("status"),
        py::arg("acc_region_elems") = 0);
  m.def("scatter_accumulate_segments", &scatter_accumulate_segments, py::arg("grads"), py::arg("chunk_numels"),
        py::arg("dst_offsets"), py::arg("acc_table"), py::arg("ctr_table"), py::arg("acc_dtype"), py::arg("my_index"),
        py::arg("scale"), py::arg("check") = false, py::arg("status") = py::none(), py::arg("acc_region_elems") = 0);
  m.def("wait_counter", &wait_counter);
  m.def("post_counts", &post_counts);
  m.def("wait_posted", &wait_posted);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd, py::arg("dy"), py::arg("x"), py::arg("w"), py::arg("rstd"),
        py::arg("fixed_order") = false, py::arg("dres") = py::none());
  m.def("rope_qkv", &rope_qkv);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("ce_fwd_bwd", &ce_fwd_bwd);
  m.def("token_logprobs", &token_logprobs);
  m.def("adamw_step", &adamw_step);
  m.def("cast_f32_to_bf16", &cast_f32_to_bf16);
  m.def("sumsq", &sumsq);
  m.def("gemm", &gemm, py::arg("a"), py::arg("b"), py::arg("c"), py::arg("layout"), py::arg("bias"),
        py::arg("accumulate"), py::arg("residual") = py::none(), py::arg("pair") = -1);
  m.def("put_block", &put_block);
  m.def("get_block", &get_block);
  m.def("scalar_put_get", &scalar_put_get);
  m.def("atomic_test", &atomic_test);
  m.def("grid_barrier_test", &grid_barrier_test);
  m.def("gemm_wgrad_scatter", &gemm_wgrad_scatter);
  m.def("gemm_wgrad_scatter_tma", &gemm_wgrad_scatter_tma, py::arg("dy"), py::arg("x"), py::arg("acc_addrs"),
        py::arg("ctr_table"), py::arg("acc_offset"), py::arg("rows_per_rank"), py::arg("scale"), py::arg("start_rank") = 0);
  m.def("gemm_gather", &gemm_gather, py::arg("x"), py::arg("shard_table"), py::arg("w_local"), py::arg("bias"),
        py::arg("rows_per_rank"), py::arg("start_rank"), py::arg("residual") = py::none());
  m.def("gemm_gather_dgrad", &gemm_gather_dgrad, py::arg("dy"), py::arg("shard_table"), py::arg("w_local"),
        py::arg("rows_per_rank"), py::arg("start_rank") = 0);
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
  m.def("kernel_status", &kernel_status);
  m.def("sm_count", &sm_count);
}
