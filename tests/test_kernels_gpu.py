"""CUDA kernels against plain PyTorch fp32 references (single GPU; peers emulated by local buffers)."""
import math
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

# The fused GEMMs can start their walk over the owners at the calling rank's own rows (off by default, read once per
# process).  Switched on here so that the emulated-rank cases below, which pass non-zero positions, cover the rotated
# tile, fetch and k orders; position 0 and the other test files cover the unrotated order.
os.environ.setdefault("ODC_GEMM_ROTATE", "2")


@pytest.fixture(scope="module")
def ext():
    from odc_b200 import _ext
    return _ext.load()


def _table(tensors):
    return torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device="cuda")


@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("n", [8, 1000, 4096 * 33 + 8, 1 << 20])
@pytest.mark.parametrize("src,dst", [(torch.bfloat16, torch.bfloat16), (torch.float32, torch.float32),
                                     (torch.float32, torch.bfloat16), (torch.int64, torch.int64)])
def test_gather_emulated_ranks(ext, world, n, src, dst):
    g = torch.Generator(device="cuda").manual_seed(n + world)
    if src == torch.int64:
        shards = [torch.randint(-2**40, 2**40, (n,), device="cuda", generator=g) for _ in range(world)]
    else:
        shards = [torch.randn(n, device="cuda", generator=g).to(src) for _ in range(world)]
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    for me in range(world):
        out = torch.empty(world, n, dtype=dst, device="cuda")
        ext.gather(out, _table(shards), n, src, me, True, status)
        want = torch.stack(shards).to(dst)
        assert torch.equal(out, want)
    assert int(status[0]) == 0


def test_gather_unaligned_rows(ext):
    world, n = 3, 1001  # 2002-byte rows: not a multiple of 16
    shards = [torch.randn(n, device="cuda").bfloat16() for _ in range(world)]
    out = torch.empty(world, n, dtype=torch.bfloat16, device="cuda")
    ext.gather(out, _table(shards), n, torch.bfloat16, 1, False, torch.zeros(4, dtype=torch.int32, device="cuda"))
    assert torch.equal(out, torch.stack(shards))


@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("n", [4, 1000, 4096 * 9 + 4, 1 << 19, 1001])
@pytest.mark.parametrize("in_dtype,acc_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32),
                                                (torch.bfloat16, torch.bfloat16)])
def test_scatter_accumulate_emulated_ranks(ext, world, n, in_dtype, acc_dtype):
    """Every emulated rank adds its [world, n] rows into the owners; sums are exactly representable."""
    if n % 2 and acc_dtype == torch.bfloat16 and world > 1:
        pytest.skip("odd bf16 rows use the scalar path tested with world 1")
    g = torch.Generator(device="cuda").manual_seed(7)
    accs = [torch.zeros(n, dtype=acc_dtype, device="cuda") for _ in range(world)]
    ctrs = [torch.zeros(8, dtype=torch.int64, device="cuda") for _ in range(world)]
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    inputs = [torch.randint(-4, 5, (world, n), device="cuda", generator=g).to(in_dtype) for _ in range(world)]
    for rounds in range(2):
        for me in range(world):
            ext.scatter_accumulate(inputs[me], _table(accs), _table(ctrs), n, acc_dtype, me, 1.0, True, status)
    want = 2 * torch.stack(inputs).float().sum(0)  # [world, n]: row p belongs to owner p
    for p in range(world):
        assert torch.equal(accs[p].float(), want[p]), (p, (accs[p].float() - want[p]).abs().max())
        assert int(ctrs[p][0]) == 2 * world
    # the arrival wait succeeds at the dispatched count ...
    ext.wait_counter(ctrs[0], 2 * world, 1000, status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    # ... and a count that nothing will ever deliver runs out of budget and reports, instead of hanging
    ext.wait_counter(ctrs[0], 2 * world + 1, 50, status)
    torch.cuda.synchronize()
    assert status[:3].tolist() == [1, 0, 2 * world]
    from odc_b200.runtime.status import OdcTimeoutError, check_status_word
    with pytest.raises(OdcTimeoutError):
        check_status_word(*status[:3].tolist())


def test_scatter_accumulate_scale(ext):
    n, world = 4096, 4
    accs = [torch.zeros(n, device="cuda") for _ in range(world)]
    ctrs = [torch.zeros(8, dtype=torch.int64, device="cuda") for _ in range(world)]
    x = torch.randint(-8, 8, (world, n), device="cuda").float()
    ext.scatter_accumulate(x, _table(accs), _table(ctrs), n, torch.float32, 0, 0.25, False,
                           torch.zeros(4, dtype=torch.int32, device="cuda"))
    assert torch.equal(torch.stack(accs), x * 0.25)


# ------------------------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("rows,cols", [(1, 256), (333, 2048), (4096, 5120), (17, 8192)])
def test_rmsnorm(rows, cols):
    from odc_b200 import ops
    from odc_b200.ops import reference as ref
    x = torch.randn(rows, cols, device="cuda").bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).bfloat16().requires_grad_()
    y = ops.rms_norm(x, w, 1e-5)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = ref.rms_norm(xr, wr, 1e-5)
    yr.backward(dy.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=2e-2, atol=2e-2 * math.sqrt(rows))


@pytest.mark.parametrize("nq,nkv,d", [(4, 4, 64), (32, 8, 64), (40, 8, 128)])
def test_rope(nq, nkv, d):
    from odc_b200 import ops
    from odc_b200.ops import reference as ref
    T = 257
    qkv = torch.randn(T, (nq + 2 * nkv) * d, device="cuda").bfloat16().requires_grad_()
    pos = torch.randint(0, 30000, (T,), device="cuda")
    out = ops.rope_qkv(qkv, pos, nq, nkv, d, 500000.0)
    dout = torch.randn_like(out)
    out.backward(dout)
    x = qkv.detach().float().cpu().requires_grad_()
    q, k, v = x.split([nq * d, nkv * d, nkv * d], dim=-1)
    want = torch.cat([ref.rope(q.reshape(T, nq, d), pos.cpu(), 500000.0).reshape(T, -1),
                      ref.rope(k.reshape(T, nkv, d), pos.cpu(), 500000.0).reshape(T, -1), v], dim=-1)
    want.backward(dout.float().cpu())
    torch.testing.assert_close(out.float().cpu(), want, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(qkv.grad.float().cpu(), x.grad, rtol=2e-2, atol=2e-2)


def test_swiglu():
    from odc_b200 import ops
    from odc_b200.ops import reference as ref
    gu = torch.randn(513, 2 * 1376, device="cuda").bfloat16().requires_grad_()
    y = ops.swiglu(gu)
    dy = torch.randn_like(y)
    y.backward(dy)
    g = gu.detach().float().requires_grad_()
    yr = ref.swiglu(g)
    yr.backward(dy.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(gu.grad.float(), g.grad, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("T,V", [(100, 1024), (300, 128256)])
def test_ce_fwd_bwd(ext, T, V):
    logits = (3 * torch.randn(T, V, device="cuda")).bfloat16()
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[5] = -100
    scale = torch.rand(T, device="cuda")
    lf = logits.float().requires_grad_()
    keep = labels != -100
    want = (torch.nn.functional.cross_entropy(lf, labels, reduction="none", ignore_index=-100) * scale).sum()
    want.backward()
    loss = torch.zeros((), device="cuda")
    ext.ce_fwd_bwd(logits, labels, scale, loss, -100)
    torch.testing.assert_close(loss, want.detach(), rtol=1e-3, atol=1e-3)
    torch.testing.assert_close(logits.float(), lf.grad, rtol=2e-2, atol=1e-4)
    assert float(logits[~keep].abs().sum()) == 0.0


def test_token_logprobs_kernel_reads_only(ext):
    """Forward-only instantiation of the cross-entropy kernel: per-row log-probability of the label, 0 for ignored
    rows, logits left untouched."""
    T, V = 300, 1000
    logits = (3 * torch.randn(T, V, device="cuda")).bfloat16()
    keep = logits.clone()
    labels = torch.randint(0, V, (T,), device="cuda")
    labels[::7] = -100
    out = torch.full((T,), 7.0, device="cuda")
    ext.token_logprobs(logits, labels, out, -100)
    want = logits.float().log_softmax(-1).gather(-1, labels.clamp_min(0)[:, None]).squeeze(-1)
    want = torch.where(labels != -100, want, torch.zeros_like(want))
    torch.testing.assert_close(out, want, rtol=1e-4, atol=2e-4)
    assert torch.equal(logits, keep)


def test_adamw_matches_torch(ext):
    n = 100003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    ref_p = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m, v, low = torch.zeros_like(p), torch.zeros_like(p), torch.empty(n, dtype=torch.bfloat16, device="cuda")
    for step in range(1, 4):
        ref_p.grad = g * step
        opt.step()
        ext.adamw_step(p, g * step, m, v, low, 1e-2, 0.9, 0.95, 1e-8, 0.1, step, 1.0)
    torch.testing.assert_close(p, ref_p.detach(), rtol=1e-5, atol=1e-6)
    assert torch.equal(low, p.bfloat16())


# ------------------------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 1376, 200), (1000, 264, 1032),
                                   (4096, 2048, 4096)])
def test_gemm_layouts(ext, layout, M, N, K):
    K = (K + 7) // 8 * 8 if layout != "tn" else K
    M = (M + 7) // 8 * 8 if layout == "tn" else M
    torch.manual_seed(M + N + K)
    A = torch.randn(M, K, device="cuda").bfloat16()
    B = torch.randn(K, N, device="cuda").bfloat16()
    want = A.float() @ B.float()
    a = A.t().contiguous() if layout == "tn" else A
    b = B.t().contiguous() if layout == "nt" else B
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ext.gemm(a, b, c, layout, None, False)
    torch.cuda.synchronize()
    assert ext.kernel_status()[0].item() == 0
    torch.testing.assert_close(c.float(), want, rtol=2e-2, atol=2e-2 * math.sqrt(K))
    # fp32 output with accumulation and bias
    bias = torch.randn(N, device="cuda").bfloat16()
    c32 = torch.ones(M, N, device="cuda")
    ext.gemm(a, b, c32, layout, bias, True)
    torch.testing.assert_close(c32, want + 1 + bias.float(), rtol=1e-2, atol=1e-2 * math.sqrt(K))


@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (256, 512, 256), (304, 1376, 200), (1000, 264, 1032),
                                   (4096, 2048, 4096), (16384, 3072, 2048)])
def test_gemm_cta_pair_layouts(ext, layout, M, N, K):
    """The CTA-pair (cta_group::2) kernel, forced: 256 x 256 tiles split over two SMs, ragged edges in M, N and K."""
    K = (K + 7) // 8 * 8 if layout != "tn" else K
    M = (M + 7) // 8 * 8 if layout == "tn" else M
    torch.manual_seed(M + N + K)
    A = torch.randn(M, K, device="cuda").bfloat16()
    B = torch.randn(K, N, device="cuda").bfloat16()
    want = A.float() @ B.float()
    a = A.t().contiguous() if layout == "tn" else A
    b = B.t().contiguous() if layout == "nt" else B
    c = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    ext.gemm(a, b, c, layout, None, False, None, 1)
    torch.cuda.synchronize()
    assert ext.kernel_status()[0].item() == 0, ext.kernel_status().tolist()
    torch.testing.assert_close(c.float(), want, rtol=2e-2, atol=2e-2 * math.sqrt(K))
    # bias + residual in the epilogue of a bf16 output
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    ext.gemm(a, b, c, layout, bias, False, res, 1)
    torch.testing.assert_close(c.float(), want + bias.float() + res.float(), rtol=2e-2, atol=2e-2 * math.sqrt(K))
    # fp32 output with accumulation (TMA reduce-add) and bias
    c32 = torch.ones(M, N, device="cuda")
    ext.gemm(a, b, c32, layout, bias, True, None, 1)
    torch.cuda.synchronize()
    assert ext.kernel_status()[0].item() == 0, ext.kernel_status().tolist()
    torch.testing.assert_close(c32, want + 1 + bias.float(), rtol=1e-2, atol=1e-2 * math.sqrt(K))
    # fp32 output, plain store over whatever the buffer held
    c32.fill_(float("nan"))
    ext.gemm(a, b, c32, layout, None, False, None, 1)
    torch.testing.assert_close(c32, want, rtol=1e-2, atol=1e-2 * math.sqrt(K))


def test_linear_autograd_matches_reference():
    from odc_b200 import ops
    x = torch.randn(3, 100, 512, device="cuda").bfloat16().requires_grad_()
    w = (0.05 * torch.randn(768, 512, device="cuda")).bfloat16().requires_grad_()
    b = torch.randn(768, device="cuda").bfloat16().requires_grad_()
    y = ops.linear(x, w, b)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(dy.float())
    torch.testing.assert_close(y.float(), yr, rtol=2e-2, atol=5e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad, rtol=2e-2, atol=5e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=2e-2, atol=0.5)
    torch.testing.assert_close(b.grad.float(), br.grad, rtol=2e-2, atol=0.5)


def test_linear_cross_entropy_matches_reference():
    from odc_b200 import ops
    from odc_b200.ops import reference as ref
    T, H, V = 700, 256, 1024
    h = torch.randn(T, H, device="cuda").bfloat16().requires_grad_()
    w = (0.05 * torch.randn(V, H, device="cuda")).bfloat16().requires_grad_()
    labels = torch.randint(0, V, (T,), device="cuda")
    scale = torch.rand(T, device="cuda") / T
    loss = ops.linear_cross_entropy(h, w, labels, scale, chunk=256)
    (loss * 2.0).backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr_ = ref.linear_cross_entropy(hr, wr, labels, scale)
    (lr_ * 2.0).backward()
    torch.testing.assert_close(loss, lr_.detach(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(h.grad.float(), hr.grad, rtol=5e-2, atol=2e-4)
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=5e-2, atol=2e-4)


@pytest.mark.parametrize("temperature", [1.0, 0.7])
def test_linear_token_logprobs_matches_reference(temperature):
    """Per-token log-probabilities and both gradients against the fp32 statement of the same head; a 3-D input,
    a ragged last chunk and ignored positions included."""
    from odc_b200 import ops
    from odc_b200.ops import reference as ref
    B, S, H, V = 2, 333, 256, 1024
    h = torch.randn(B, S, H, device="cuda").bfloat16().requires_grad_()
    w = (0.05 * torch.randn(V, H, device="cuda")).bfloat16().requires_grad_()
    ids = torch.randint(0, V, (B, S), device="cuda")
    ids[0, :5] = -100
    adv = torch.randn(B, S, device="cuda")
    lp = ops.linear_token_logprobs(h, w, ids, temperature, chunk=256)
    assert lp.shape == ids.shape and lp.dtype == torch.float32
    (lp * adv).sum().backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lpr = ref.linear_token_logprobs(hr.view(-1, H), wr, ids.view(-1), temperature).view(B, S)
    (lpr * adv).sum().backward()
    assert float(lp[0, :5].abs().max()) == 0.0
    torch.testing.assert_close(lp, lpr.detach(), rtol=2e-2, atol=3e-2)
    torch.testing.assert_close(h.grad.float(), hr.grad, rtol=5e-2, atol=3e-2)
    torch.testing.assert_close(w.grad.float(), wr.grad, rtol=5e-2, atol=5e-2)
    assert float(h.grad[0, :5].float().abs().max()) == 0.0


# ------------------------------------------------------------------------------------ fused compute + comm
@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("T,n_out,k_in", [(512, 256, 256), (1000, 768, 264), (4096, 2048, 2048)])
def test_wgrad_scatter_emulated_ranks(ext, world, T, n_out, k_in):
    """dW = dY^T X reduced straight into per-owner fp32 accumulators (owners emulated by local buffers)."""
    torch.manual_seed(T + n_out)
    rows_per = (n_out + world - 1) // world
    off = 64  # the parameter starts 64 elements into each accumulator
    accs = [torch.zeros(off + rows_per * k_in + 32, device="cuda") for _ in range(world)]
    ctrs = [torch.zeros(8, dtype=torch.int64, device="cuda") for _ in range(world)]
    want = torch.zeros(n_out, k_in, device="cuda")
    for producer in range(2):  # two emulated producers add into the same owners
        dy = torch.randn(T, n_out, device="cuda").bfloat16()
        x = torch.randn(T, k_in, device="cuda").bfloat16()
        ext.gemm_wgrad_scatter(dy, x, _table(accs), _table(ctrs), off, rows_per, 0.5)
        want += 0.5 * (dy.float().t() @ x.float())
    torch.cuda.synchronize()
    assert ext.kernel_status()[0].item() == 0
    for r in range(world):
        rows = max(0, min(rows_per, n_out - r * rows_per))
        got = accs[r][off:off + rows * k_in].view(rows, k_in)
        torch.testing.assert_close(got, want[r * rows_per:r * rows_per + rows], rtol=2e-2, atol=2e-2 * math.sqrt(T))
        assert float(accs[r][:off].abs().sum()) == 0.0 and float(accs[r][off + rows_per * k_in:].abs().sum()) == 0.0
        assert int(ctrs[r][0]) == 2


@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (1000, 1376, 512), (8192, 3072, 2048), (300, 264, 128)])
def test_gemm_gather_emulated_ranks(ext, world, M, N, K):
    """Y = X W^T with W assembled from row shards while the GEMM runs (owners emulated by local buffers)."""
    torch.manual_seed(M + N + K)
    rows_per = (N + world - 1) // world
    W = torch.randn(world * rows_per, K, device="cuda").bfloat16()
    shards = [W[r * rows_per:(r + 1) * rows_per].clone() for r in range(world)]
    x = torch.randn(M, K, device="cuda").bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    w_local = torch.zeros(N, K, dtype=torch.bfloat16, device="cuda")
    y = ext.gemm_gather(x, _table(shards), w_local, bias, rows_per, (world - 1) if world > 2 else 1 % world)
    torch.cuda.synchronize()
    assert ext.kernel_status()[0].item() == 0, ext.kernel_status().tolist()
    assert torch.equal(w_local, W[:N])
    torch.testing.assert_close(y.float(), x.float() @ W[:N].float().t() + bias.float(), rtol=2e-2, atol=2e-2 * math.sqrt(K))


@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (1000, 1376, 512), (8192, 3072, 2048), (300, 264, 128)])
def test_gemm_gather_dgrad_emulated_ranks(ext, world, M, N, K):
    """dX = dY W with W's rows (the reduction dimension) assembled from shards while the GEMM runs."""
    torch.manual_seed(M + N + K + 1)
    rows_per = (N + world - 1) // world
    W = (0.1 * torch.randn(world * rows_per, K, device="cuda")).bfloat16()
    shards = [W[r * rows_per:(r + 1) * rows_per].clone() for r in range(world)]
    dy = torch.randn(M, N, device="cuda").bfloat16()
    w_local = torch.zeros(N, K, dtype=torch.bfloat16, device="cuda")
    dx = ext.gemm_gather_dgrad(dy, _table(shards), w_local, rows_per, (world * 5 + 3) % world if world > 2 else world - 1)
    torch.cuda.synchronize()
    assert ext.kernel_status()[0].item() == 0, ext.kernel_status().tolist()
    assert torch.equal(w_local, W[:N])
    torch.testing.assert_close(dx.float(), dy.float() @ W[:N].float(), rtol=2e-2, atol=2e-2 * math.sqrt(N) * 0.1)


def test_linear_with_fused_residual():
    from odc_b200 import ops
    x = torch.randn(300, 512, device="cuda").bfloat16().requires_grad_()
    w = (0.05 * torch.randn(768, 512, device="cuda")).bfloat16().requires_grad_()
    res = torch.randn(300, 768, device="cuda").bfloat16().requires_grad_()
    y = ops.linear(x, w, None, residual=res)
    dy = torch.randn_like(y)
    y.backward(dy)
    want = x.detach().float() @ w.detach().float().t() + res.detach().float()
    torch.testing.assert_close(y.float(), want, rtol=2e-2, atol=5e-2)
    assert torch.equal(res.grad, dy)


@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("T,n_out,k_in", [(512, 1024, 256), (1000, 2048, 264), (4096, 2048, 2048)])
def test_wgrad_scatter_tma_emulated_ranks(ext, world, T, n_out, k_in):
    """Same contract as the red.add variant, output through smem staging + TMA reduce-add (owners emulated locally)."""
    torch.manual_seed(T + n_out)
    rows_per = (n_out + world - 1) // world
    rows_per = (rows_per + 127) // 128 * 128
    off = 64
    accs = [torch.zeros(off + rows_per * k_in + 32, device="cuda") for _ in range(world)]
    ctrs = [torch.zeros(8, dtype=torch.int64, device="cuda") for _ in range(world)]
    want = torch.zeros(world * rows_per, k_in, device="cuda")
    for producer in range(2):
        dy = torch.randn(T, n_out, device="cuda").bfloat16()
        x = torch.randn(T, k_in, device="cuda").bfloat16()
        # the producer's position in the group only rotates the order in which the owners' tiles are produced
        assert ext.gemm_wgrad_scatter_tma(dy, x, [a.data_ptr() for a in accs], _table(ctrs), off, rows_per, 0.5,
                                          (producer * 5 + 1) % world)
        want[:n_out] += 0.5 * (dy.float().t() @ x.float())
    torch.cuda.synchronize()
    assert ext.kernel_status()[0].item() == 0
    for r in range(world):
        got = accs[r][off:off + rows_per * k_in].view(rows_per, k_in)
        torch.testing.assert_close(got, want[r * rows_per:(r + 1) * rows_per], rtol=2e-2, atol=2e-2 * math.sqrt(T))
        assert float(accs[r][:off].abs().sum()) == 0.0 and float(accs[r][off + rows_per * k_in:].abs().sum()) == 0.0
        assert int(ctrs[r][0]) == 2
    # ineligible split (rows per owner not a multiple of 128): the entry point declines, nothing is launched
    assert not ext.gemm_wgrad_scatter_tma(dy, x, [a.data_ptr() for a in accs], _table(ctrs), off, 100, 1.0)


def test_scatter_accumulate_bulk_path_matches(ext):
    """The opt-in bulk (TMA) scatter path gives the same sums; run in a child process so the switch is seen at first use."""
    import subprocess, sys, os, textwrap
    code = textwrap.dedent("""
        import torch, sys
        sys.path.insert(0, %r)
        from odc_b200 import _ext
        ext = _ext.load()
        world, n = 4, 1 << 18
        accs = [torch.zeros(n, device="cuda") for _ in range(world)]
        ctrs = [torch.zeros(8, dtype=torch.int64, device="cuda") for _ in range(world)]
        tab = lambda ts: torch.tensor([t.data_ptr() for t in ts], dtype=torch.int64, device="cuda")
        xs = [torch.randint(-4, 5, (world, n), device="cuda").float() for _ in range(world)]
        st = torch.zeros(4, dtype=torch.int32, device="cuda")
        for me in range(world):
            ext.scatter_accumulate(xs[me], tab(accs), tab(ctrs), n, torch.float32, me, 1.0, False, st)
        torch.cuda.synchronize()
        want = torch.stack(xs).sum(0)
        assert all(torch.equal(accs[p], want[p]) for p in range(world))
        assert all(int(c[0]) == world for c in ctrs) and int(st[0]) == 0
        print("BULK_OK")
    """ % os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    r = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, ODC_SCATTER_BULK="1"), capture_output=True, text=True,
                       timeout=120)
    assert r.returncode == 0 and "BULK_OK" in r.stdout, r.stdout + r.stderr


@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_scatter_accumulate_segments_emulated_ranks(ext, world, dtype):
    """Reduction straight from a list of gradient tensors: same result as flattening them rank-major first."""
    torch.manual_seed(world)
    shapes = [(1024, 512), (512,), (300, 96), (7, 5), (world * 3 + 1, 64), (2048, 2048)]
    grads = [torch.randn(*s, device="cuda").to(dtype) for s in shapes]
    chunks, offsets, o = [], [], 0
    for g in grads:
        rows = -(-g.shape[0] // world)
        c = rows * (g.numel() // g.shape[0])
        chunks.append(c)
        offsets.append(o)
        o += c
    accs = [torch.zeros(o + 16, device="cuda") for _ in range(world)]
    ctrs = [torch.zeros(8, dtype=torch.int64, device="cuda") for _ in range(world)]
    for _ in range(2):
        assert ext.scatter_accumulate_segments(grads, chunks, offsets, _table(accs), _table(ctrs), torch.float32, 1 % world, 0.5)
    torch.cuda.synchronize()
    for r in range(world):
        want = torch.zeros(o + 16, device="cuda")
        for g, c, off in zip(grads, chunks, offsets):
            piece = g.reshape(-1)[r * c:(r + 1) * c].float()
            want[off:off + piece.numel()] += 2 * 0.5 * piece
        torch.testing.assert_close(accs[r], want, rtol=1e-6, atol=1e-6)
        assert int(ctrs[r][0]) == 2
    # lists this path does not take are refused without a launch
    assert not ext.scatter_accumulate_segments([grads[0]] * 33, [chunks[0]] * 33, [0] * 33, _table(accs), _table(ctrs),
                                               torch.float32, 0, 1.0)
    assert not ext.scatter_accumulate_segments(grads, chunks, offsets, _table(accs), _table(ctrs), torch.bfloat16, 0, 1.0)


# ------------------------------------------------------------------------------------ debug bounds checks
def test_debug_bounds_refuse_a_short_declared_region(ext):
    """ODC_DEBUG_BOUNDS launches: a row longer than the DECLARED region is refused on valid memory.

    Every buffer here is fully allocated, only the declared length is made too short, so nothing out of range
    is ever touched; a refused launch leaves the destination untouched and reports through the status word.
    """
    world, n = 2, 4096
    from odc_b200.runtime.status import ERR_BOUNDS, ERR_PEER_INDEX
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    # gather
    shards = [torch.ones(n, device="cuda").bfloat16() * (r + 1) for r in range(world)]
    out = torch.zeros(world, n, dtype=torch.bfloat16, device="cuda")
    ext.gather(out, _table(shards), n, torch.bfloat16, 0, True, status, n - 8)
    torch.cuda.synchronize()
    assert int(status[0]) == ERR_BOUNDS and float(out.abs().sum()) == 0
    status.zero_()
    ext.gather(out, _table(shards), n, torch.bfloat16, 5, True, status, n)      # start index outside the group
    torch.cuda.synchronize()
    assert int(status[0]) == ERR_PEER_INDEX and float(out.abs().sum()) == 0
    status.zero_()
    ext.gather(out, _table(shards), n, torch.bfloat16, 1, True, status, n)      # exact fit passes
    torch.cuda.synchronize()
    assert int(status[0]) == 0 and torch.equal(out, torch.stack(shards))
    # scatter_accumulate (fp32 and bf16 sources, fp32 and bf16 accumulators)
    for in_dtype, acc_dtype in [(torch.float32, torch.float32), (torch.bfloat16, torch.float32),
                                (torch.bfloat16, torch.bfloat16)]:
        accs = [torch.zeros(n, dtype=acc_dtype, device="cuda") for _ in range(world)]
        ctrs = [torch.zeros(8, dtype=torch.int64, device="cuda") for _ in range(world)]
        x = torch.ones(world, n, device="cuda").to(in_dtype)
        status.zero_()
        ext.scatter_accumulate(x, _table(accs), _table(ctrs), n, acc_dtype, 0, 1.0, True, status, n - 4)
        torch.cuda.synchronize()
        assert int(status[0]) == ERR_BOUNDS
        assert all(float(a.float().abs().sum()) == 0 for a in accs)
        assert all(int(c[0]) == 1 for c in ctrs)   # the owners are not left waiting for the refused contribution
        status.zero_()
        ext.scatter_accumulate(x, _table(accs), _table(ctrs), n, acc_dtype, 0, 1.0, True, status, n)
        torch.cuda.synchronize()
        assert int(status[0]) == 0 and all(float(a.float().sum()) == n for a in accs)
    # segmented scatter: the second tensor would end past the declared accumulator length
    accs = [torch.zeros(3 * n, device="cuda") for _ in range(world)]
    ctrs = [torch.zeros(8, dtype=torch.int64, device="cuda") for _ in range(world)]
    grads = [torch.ones(world * n, device="cuda"), torch.ones(world * 2 * n, device="cuda")]
    status.zero_()
    assert ext.scatter_accumulate_segments(grads, [n, 2 * n], [0, n], _table(accs), _table(ctrs), torch.float32, 0, 1.0,
                                           True, status, 3 * n - 4)
    torch.cuda.synchronize()
    assert int(status[0]) == ERR_BOUNDS and all(float(a.sum()) == 0 for a in accs)
    status.zero_()
    assert ext.scatter_accumulate_segments(grads, [n, 2 * n], [0, n], _table(accs), _table(ctrs), torch.float32, 0, 1.0,
                                           True, status, 3 * n)
    torch.cuda.synchronize()
    assert int(status[0]) == 0 and all(float(a.sum()) == 3 * n for a in accs)


def test_posted_counts_and_bounded_wait(ext):
    """One-sided dispatch-count exchange, with the producers emulated by separate posts into one owner's slots."""
    nprod = 5
    slots = torch.zeros(8, dtype=torch.int64, device="cuda")
    ctr = torch.zeros(8, dtype=torch.int64, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    expected = torch.zeros(1, dtype=torch.int64, device="cuda")
    counts = [3, 0, 7, 1, 2]
    for p, c in enumerate(counts):
        ext.post_counts([slots.data_ptr() + 8 * p], [c], 1, 0)
    ctr[0] = sum(counts)
    ext.wait_posted(slots, nprod, 1, ctr, 500, status, expected)
    torch.cuda.synchronize()
    assert int(status[0]) == 0 and int(expected[0]) == sum(counts)
    assert [int(v) >> 32 for v in slots[:nprod]] == [1] * nprod
    # a synchronisation that one producer never posts for: the wait runs out and names the producer
    for p, c in enumerate(counts[:-1]):
        ext.post_counts([slots.data_ptr() + 8 * p], [c + 1], 2, 0)
    ext.wait_posted(slots, nprod, 2, ctr, 50, status, expected)
    torch.cuda.synchronize()
    assert status[:3].tolist() == [1, 1000 + nprod - 1, 1]
    # all postings there, but fewer arrivals than announced: the arrival wait runs out instead
    status.zero_()
    ext.post_counts([slots.data_ptr() + 8 * (nprod - 1)], [counts[-1] + 1], 2, 0)
    ext.wait_posted(slots, nprod, 2, ctr, 50, status, expected)
    torch.cuda.synchronize()
    assert status[:3].tolist() == [1, 0, sum(counts)] and int(expected[0]) == sum(counts) + nprod


def test_rmsnorm_residual_backward_fuses_the_residual_gradient():
    """(norm(x), x): the gradient of the pass-through output is added inside the norm's backward kernel."""
    from odc_b200 import ops
    rows, cols = 777, 2048
    x = torch.randn(rows, cols, device="cuda").bfloat16().requires_grad_()
    w = (1 + 0.1 * torch.randn(cols, device="cuda")).bfloat16().requires_grad_()
    y, xr = ops.rms_norm_residual(x, w, 1e-5)
    dy, dres = torch.randn_like(y), torch.randn_like(xr)
    torch.autograd.backward([y, xr], [dy, dres])
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
    torch.autograd.backward([yf, xf * 1.0], [dy.float(), dres.float()])
    torch.testing.assert_close(y.float(), yf, rtol=2e-2, atol=2e-2)
    assert xr.data_ptr() == x.data_ptr()
    torch.testing.assert_close(x.grad.float(), xf.grad, rtol=2e-2, atol=3e-2)
    torch.testing.assert_close(w.grad.float(), wf.grad, rtol=2e-2, atol=rows ** 0.5 * 2e-2)
    # only the normalised branch is used: the pass-through gradient is absent
    x2 = x.detach().clone().requires_grad_()
    y2, _ = ops.rms_norm_residual(x2, w.detach(), 1e-5)
    y2.backward(dy)
    xg = x.detach().float().requires_grad_()
    (xg * torch.rsqrt(xg.pow(2).mean(-1, keepdim=True) + 1e-5) * w.detach().float()).backward(dy.float())
    torch.testing.assert_close(x2.grad.float(), xg.grad, rtol=2e-2, atol=3e-2)
