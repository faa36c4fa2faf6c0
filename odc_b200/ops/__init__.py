"""Differentiable ops of the decoder.

On CUDA every op runs this package's own sm_100a kernels through the native extension (and
raises if the extension is missing); on CPU the plain PyTorch statements in
:mod:`odc_b200.ops.reference` run instead, which is what the CPU/gloo tests use.

``ODC_GEMM=cublas`` and ``ODC_ATTN=flash`` switch the two largest kernels to library calls; they
exist to measure the hand-written kernels against the libraries, not as a fallback.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from . import reference as ref

_launches = 0


def kernel_launches() -> int:
    """Number of this package's kernels launched by the ops so far (for benchmark accounting)."""
    return _launches


def _count(n: int = 1):
    global _launches
    _launches += n


def _ext():
    from .. import _ext as loader
    return loader.load()


def check_status() -> None:
    """Raise if a kernel of this package gave up on a bounded wait since the last check (one small D2H copy + sync).

    The FSDP integrations and the reduction service read the same per-device word at every once-per-minibatch
    synchronisation; code that uses the ops on their own calls this where it would otherwise trust the results.
    """
    from ..runtime.status import check_status_word
    word = _ext().kernel_status()
    host = word.cpu()
    if int(host[0]) != 0:
        word.zero_()
        check_status_word(int(host[0]), int(host[1]), int(host[2]))


def gemm_backend() -> str:
    return os.environ.get("ODC_GEMM", "tcgen05")


def attn_backend() -> str:
    return os.environ.get("ODC_ATTN", "native")


# ------------------------------------------------------------------------------------------
# GEMM.  layouts (all operands row-major):
#   "nt": C[M,N] = A[M,K] @ B[N,K]^T      (forward  y = x W^T)
#   "nn": C[M,N] = A[M,K] @ B[K,N]        (dgrad    dx = dy W)
#   "tn": C[M,N] = A[K,M]^T @ B[K,N]      (wgrad    dW = dy^T x)
# ------------------------------------------------------------------------------------------
def gemm(a: torch.Tensor, b: torch.Tensor, layout: str = "nt", out: Optional[torch.Tensor] = None,
         bias: Optional[torch.Tensor] = None, out_dtype: Optional[torch.dtype] = None,
         accumulate: bool = False, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    if layout == "nt":
        M, N = a.shape[0], b.shape[0]
    elif layout == "nn":
        M, N = a.shape[0], b.shape[1]
    elif layout == "tn":
        M, N = a.shape[1], b.shape[1]
    else:
        raise ValueError(layout)
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
        assert not accumulate
    if not a.is_cuda or gemm_backend() == "cublas":
        A = a.t() if layout == "tn" else a
        B = b.t() if layout == "nt" else b
        r = (A.float() @ B.float()) if not a.is_cuda else (A @ B)
        if bias is not None:
            r = r + bias
        if residual is not None:
            r = r + residual
        if accumulate:
            out += r.to(out.dtype)
        else:
            out.copy_(r)
        return out
    _ext().gemm(a, b, out, layout, bias, accumulate, residual)
    _count()
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, residual):
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        x2 = x.reshape(-1, x.shape[-1])
        res2 = None if residual is None else residual.reshape(-1, w.shape[0])
        y = gemm(x2, w, "nt", bias=bias, residual=res2)  # the residual is added in the GEMM epilogue
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, "nn").view(x.shape)
        if ctx.needs_input_grad[1]:
            dw = gemm(dy2, x2, "tn", out_dtype=w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2.float().sum(0).to(dy.dtype)
        dres = dy if ctx.needs_input_grad[3] else None
        return dx, dw, db, dres


def linear(x, w, bias=None, residual=None):
    """``x @ w.T (+ bias) (+ residual)``; on CUDA bias and residual are fused into the GEMM epilogue."""
    if not x.is_cuda:
        y = ref.linear(x, w, bias)
        return y if residual is None else y + residual
    return _Linear.apply(x, w, bias, residual)


# ------------------------------------------------------------------------------------------
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        x2 = x.reshape(-1, x.shape[-1])
        y, rstd = _ext().rmsnorm_fwd(x2, weight, eps)
        _count()
        ctx.save_for_backward(x2, weight, rstd)
        ctx.shape = x.shape
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, rstd = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        from .. import config
        fixed = config.deterministic()   # fixed-order column sums (two launches) instead of in-kernel atomics (one)
        dx, dw = _ext().rmsnorm_bwd(dy2, x2, weight, rstd, fixed)
        _count(2 if fixed else 1)
        return dx.view(ctx.shape), dw.to(weight.dtype), None


def rms_norm(x, weight, eps: float = 1e-6):
    if not x.is_cuda:
        return ref.rms_norm(x, weight, eps)
    return _RMSNorm.apply(x.contiguous(), weight, eps)


class _RMSNormResidual(torch.autograd.Function):
    """``(rms_norm(x), x)``: the second output carries the residual stream.  Its gradient and the normalised
    branch's gradient meet again in backward, where ONE kernel forms ``d rms_norm + d residual`` (autograd would
    otherwise add the two with a separate full pass over the activation)."""

    @staticmethod
    def forward(ctx, x, weight, eps):
        x2 = x.reshape(-1, x.shape[-1])
        y, rstd = _ext().rmsnorm_fwd(x2, weight, eps)
        _count()
        ctx.save_for_backward(x2, weight, rstd)
        ctx.shape = x.shape
        return y.view(x.shape), x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dres):
        x2, weight, rstd = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dr2 = None if dres is None else dres.reshape(-1, dres.shape[-1]).contiguous()
        from .. import config
        fixed = config.deterministic()
        dx, dw = _ext().rmsnorm_bwd(dy2, x2, weight, rstd, fixed, dr2)
        _count(2 if fixed else 1)
        return dx.view(ctx.shape), dw.to(weight.dtype), None


def rms_norm_residual(x, weight, eps: float = 1e-6):
    """``(rms_norm(x, weight), x)`` for pre-norm blocks: feed the second value to the block's residual add."""
    if not x.is_cuda:
        return ref.rms_norm(x, weight, eps), x
    return _RMSNormResidual.apply(x.contiguous(), weight, eps)


# ------------------------------------------------------------------------------------------
class _Rope(torch.autograd.Function):
    """Rotary embedding applied to the q and k heads of a fused ``[T, (Hq+2Hkv)*D]`` projection."""

    @staticmethod
    def forward(ctx, qkv, position_ids, n_q, n_kv, head_dim, theta):
        ctx.save_for_backward(position_ids)
        ctx.cfg = (n_q, n_kv, head_dim, theta)
        out = _ext().rope_qkv(qkv, position_ids, n_q, n_kv, head_dim, theta, False)
        _count()
        return out

    @staticmethod
    def backward(ctx, dout):
        (position_ids,) = ctx.saved_tensors
        n_q, n_kv, head_dim, theta = ctx.cfg
        dqkv = _ext().rope_qkv(dout.contiguous(), position_ids, n_q, n_kv, head_dim, theta, True)
        _count()
        return dqkv, None, None, None, None, None


def rope_qkv(qkv, position_ids, n_q: int, n_kv: int, head_dim: int, theta: float,
             inv_freq: Optional[torch.Tensor] = None):
    """Rotate the q and k parts of a fused qkv activation; v passes through.

    ``inv_freq`` (rescaled rotary frequencies, ``ops.reference.rope_inv_freq``) selects the PyTorch statements on
    any device: the kernel derives its frequencies from ``theta`` alone.
    """
    if not qkv.is_cuda or inv_freq is not None:
        T = qkv.shape[0]
        q, k, v = qkv.split([n_q * head_dim, n_kv * head_dim, n_kv * head_dim], dim=-1)
        q = ref.rope(q.reshape(T, n_q, head_dim), position_ids, theta, inv_freq=inv_freq).reshape(T, -1)
        k = ref.rope(k.reshape(T, n_kv, head_dim), position_ids, theta, inv_freq=inv_freq).reshape(T, -1)
        return torch.cat([q, k, v], dim=-1)
    return _Rope.apply(qkv, position_ids, n_q, n_kv, head_dim, theta)


# ------------------------------------------------------------------------------------------
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        ctx.save_for_backward(gate_up)
        y = _ext().swiglu_fwd(gate_up)
        _count()
        return y

    @staticmethod
    def backward(ctx, dy):
        (gate_up,) = ctx.saved_tensors
        d = _ext().swiglu_bwd(dy.contiguous(), gate_up)
        _count()
        return d


def swiglu(gate_up):
    if not gate_up.is_cuda:
        return ref.swiglu(gate_up)
    return _SwiGLU.apply(gate_up.contiguous())


# ------------------------------------------------------------------------------------------
class _VarlenAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, max_seqlen, causal, scale):
        o, lse = _ext().attn_fwd(q, k, v, cu_seqlens, max_seqlen, causal, scale)
        _count()
        ctx.save_for_backward(q, k, v, o, lse, cu_seqlens)
        ctx.cfg = (max_seqlen, causal, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, cu_seqlens = ctx.saved_tensors
        max_seqlen, causal, scale = ctx.cfg
        dq, dk, dv, _ = _ext().attn_bwd(do.contiguous(), q, k, v, o, lse, cu_seqlens, max_seqlen, causal, scale, False)
        _count(3)
        return dq, dk, dv, None, None, None, None


class _VarlenAttentionQKV(torch.autograd.Function):
    """Attention straight on a fused ``[T, (Hq+2Hkv)*D]`` projection: q/k/v are column views in forward and the
    backward kernels write dq/dk/dv into column views of ONE gradient tensor, so autograd never materialises
    zero-padded slices."""

    @staticmethod
    def forward(ctx, qkv, n_q, n_kv, head_dim, cu_seqlens, max_seqlen, causal, scale):
        T = qkv.shape[0]
        nq, nk = n_q * head_dim, n_kv * head_dim
        q = qkv[:, :nq].view(T, n_q, head_dim)
        k = qkv[:, nq:nq + nk].view(T, n_kv, head_dim)
        v = qkv[:, nq + nk:].view(T, n_kv, head_dim)
        o, lse = _ext().attn_fwd(q, k, v, cu_seqlens, max_seqlen, causal, scale)
        _count()
        ctx.save_for_backward(qkv, o, lse, cu_seqlens)
        ctx.cfg = (n_q, n_kv, head_dim, max_seqlen, causal, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse, cu_seqlens = ctx.saved_tensors
        n_q, n_kv, head_dim, max_seqlen, causal, scale = ctx.cfg
        T = qkv.shape[0]
        nq, nk = n_q * head_dim, n_kv * head_dim
        q = qkv[:, :nq].view(T, n_q, head_dim)
        k = qkv[:, nq:nq + nk].view(T, n_kv, head_dim)
        v = qkv[:, nq + nk:].view(T, n_kv, head_dim)
        _, _, _, dqkv = _ext().attn_bwd(do.contiguous(), q, k, v, o, lse, cu_seqlens, max_seqlen, causal, scale, True)
        _count(3)
        return dqkv, None, None, None, None, None, None, None


def varlen_attention_qkv(qkv, n_q: int, n_kv: int, head_dim: int, cu_seqlens, max_seqlen: int, causal: bool = True,
                         scale: Optional[float] = None):
    """Causal attention on a fused qkv activation ``[T, (Hq+2Hkv)*D]``; returns ``[T, Hq, D]``."""
    scale = scale if scale is not None else 1.0 / math.sqrt(head_dim)
    T = qkv.shape[0]
    if qkv.is_cuda and attn_backend() == "native":
        return _VarlenAttentionQKV.apply(qkv, n_q, n_kv, head_dim, cu_seqlens, max_seqlen, causal, scale)
    nq, nk = n_q * head_dim, n_kv * head_dim
    q = qkv[:, :nq].view(T, n_q, head_dim)
    k = qkv[:, nq:nq + nk].view(T, n_kv, head_dim)
    v = qkv[:, nq + nk:].view(T, n_kv, head_dim)
    return varlen_attention(q, k, v, cu_seqlens, max_seqlen, causal, scale)


def varlen_attention(q, k, v, cu_seqlens, max_seqlen: int, causal: bool = True, scale: Optional[float] = None):
    """Causal attention over packed sequences; q ``[T,Hq,D]``, k/v ``[T,Hkv,D]`` (strided views allowed)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if not q.is_cuda:
        return ref.varlen_attention(q, k, v, cu_seqlens, causal, scale)
    if attn_backend() == "flash":
        from flash_attn import flash_attn_varlen_func
        return flash_attn_varlen_func(q, k, v, cu_seqlens, cu_seqlens, max_seqlen, max_seqlen,
                                      softmax_scale=scale, causal=causal)
    return _VarlenAttention.apply(q, k, v, cu_seqlens, max_seqlen, causal, scale)


# ------------------------------------------------------------------------------------------
class _LinearCrossEntropy(torch.autograd.Function):
    """Loss and both gradients in one pass over token chunks; ``[T, vocab]`` logits never exist.

    Same mathematics as the reference's chunked LM head (examples/llm_training/lm_head.py:7-59)
    but the gradients are formed while the chunk's logits are still on chip-adjacent memory, so
    backward is a scalar multiply instead of a second pass of GEMMs.
    """

    @staticmethod
    def forward(ctx, h, w, labels, loss_scale, ignore_index, chunk):
        T, H = h.shape
        V = w.shape[0]
        ext = _ext()
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dh = torch.empty_like(h) if need_dh else None
        dw32 = torch.empty(V, H, dtype=torch.float32, device=h.device) if need_dw else None  # written by the first chunk
        loss = torch.zeros((), dtype=torch.float32, device=h.device)
        logits = torch.empty(min(chunk, T), V, dtype=torch.bfloat16, device=h.device)
        if T == 0 and dw32 is not None:
            dw32.zero_()
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            lg = logits[: e - s]
            gemm(h[s:e], w, "nt", out=lg)
            # in place: logits -> dlogits = loss_scale * (softmax - onehot); adds the chunk's loss
            ext.ce_fwd_bwd(lg, labels[s:e], None if loss_scale is None else loss_scale[s:e], loss, ignore_index)
            _count()
            if need_dh:
                gemm(lg, w, "nn", out=dh[s:e])
            if need_dw:
                gemm(lg, h[s:e], "tn", out=dw32, accumulate=s > 0)
        ctx.save_for_backward(dh, dw32)
        ctx.w_dtype = w.dtype
        return loss

    @staticmethod
    def backward(ctx, dloss):
        dh, dw32 = ctx.saved_tensors
        gh = (dh * dloss.to(dh.dtype)) if dh is not None else None
        gw = (dw32 * dloss).to(ctx.w_dtype) if dw32 is not None else None
        return gh, gw, None, None, None, None


def linear_cross_entropy(h, w, labels, loss_scale=None, ignore_index: int = -100, chunk: int = 4096):
    """Summed (optionally per-token weighted) cross-entropy of ``h @ w.T`` against ``labels``."""
    if not h.is_cuda:
        return ref.linear_cross_entropy(h, w, labels, loss_scale, ignore_index, chunk)
    if loss_scale is not None and loss_scale.dtype != torch.float32:
        loss_scale = loss_scale.float()  # FSDP's mixed-precision input cast may have narrowed it
    return _LinearCrossEntropy.apply(h.contiguous(), w, labels.contiguous(), loss_scale, ignore_index, chunk)


class _LinearTokenLogProbs(torch.autograd.Function):
    """Per-token log-probability of ``ids`` under ``softmax(h @ w.T / temperature)``, in token chunks.

    The policy-gradient form of the chunked LM head (the reference's ``FusedLinearForPPOFunction``,
    examples/llm_training/lm_head.py:62-190).  Forward is one GEMM and one read-only pass of the cross-entropy
    kernel per chunk (one number per token comes out).  The weights of the tokens are only known in backward, so
    backward recomputes each chunk's logits, turns them in place into
    ``dlogp / temperature * (onehot - softmax)`` with the cross-entropy kernel (its per-token scale is
    ``-dlogp / temperature``) and feeds the two gradient GEMMs; ``[T, vocab]`` logits never exist.
    """

    @staticmethod
    def forward(ctx, h, w, ids, temperature, ignore_index, chunk):
        T = h.shape[0]
        V = w.shape[0]
        ext = _ext()
        out = torch.zeros(T, dtype=torch.float32, device=h.device)
        logits = torch.empty(min(chunk, T), V, dtype=torch.bfloat16, device=h.device)
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            lg = logits[: e - s]
            gemm(h[s:e], w, "nt", out=lg)
            if temperature != 1.0:
                lg.mul_(1.0 / temperature)
            ext.token_logprobs(lg, ids[s:e], out[s:e], ignore_index)   # one pass over the chunk's logits
            _count()
        ctx.save_for_backward(h, w, ids)
        ctx.args = (temperature, ignore_index, chunk)
        return out

    @staticmethod
    def backward(ctx, dlogp):
        h, w, ids = ctx.saved_tensors
        temperature, ignore_index, chunk = ctx.args
        T, H = h.shape
        V = w.shape[0]
        ext = _ext()
        need_dh, need_dw = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dh = torch.empty_like(h) if need_dh else None
        dw32 = torch.empty(V, H, dtype=torch.float32, device=h.device) if need_dw else None
        if T == 0 and dw32 is not None:
            dw32.zero_()
        scale = (dlogp.reshape(-1).float() * (-1.0 / temperature)).contiguous()
        sink = torch.zeros((), dtype=torch.float32, device=h.device)   # the kernel's loss output is not used here
        logits = torch.empty(min(chunk, T), V, dtype=torch.bfloat16, device=h.device)
        for s in range(0, T, chunk):
            e = min(T, s + chunk)
            lg = logits[: e - s]
            gemm(h[s:e], w, "nt", out=lg)
            if temperature != 1.0:
                lg.mul_(1.0 / temperature)
            ext.ce_fwd_bwd(lg, ids[s:e], scale[s:e], sink, ignore_index)
            _count()
            if need_dh:
                gemm(lg, w, "nn", out=dh[s:e])
            if need_dw:
                gemm(lg, h[s:e], "tn", out=dw32, accumulate=s > 0)
        return dh, (dw32.to(w.dtype) if dw32 is not None else None), None, None, None, None


def linear_token_logprobs(h, w, ids, temperature: float = 1.0, ignore_index: int = -100, chunk: int = 4096):
    """``log_softmax(h @ w.T / temperature)[t, ids[t]]`` as fp32, for ``h`` of shape ``[T, H]`` or ``[B, S, H]``.

    Positions whose id equals ``ignore_index`` give 0 and no gradient.
    """
    shape = ids.shape
    h2 = h.reshape(-1, h.shape[-1])
    flat = ids.reshape(-1).to(torch.int64)
    if not h.is_cuda:
        return ref.linear_token_logprobs(h2, w, flat, temperature, ignore_index, chunk).view(shape)
    return _LinearTokenLogProbs.apply(h2.contiguous(), w, flat.contiguous(), float(temperature), ignore_index,
                                      chunk).view(shape)


class LinearTokenLogProbs(torch.nn.Module):
    """Module form: ``forward(hidden_states, vocab_weights, input_ids, temperature) -> (log_probs, None)``.

    The second value is the place of the entropy the reference's module leaves unset as well
    (examples/llm_training/lm_head.py:193-214).
    """

    def __init__(self, chunk_size: int = 4096):
        super().__init__()
        self.chunk_size = chunk_size

    def forward(self, hidden_states, vocab_weights, input_ids, temperature: float = 1.0):
        return linear_token_logprobs(hidden_states, vocab_weights, input_ids, temperature, chunk=self.chunk_size), None


# ------------------------------------------------------------------------------------------
def fused_adamw_(p32, g, m, v, p_lowp, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0):
    """One AdamW step on a flat fp32 shard; also refreshes the low-precision copy that peers gather."""
    if not p32.is_cuda:
        ref.adamw_step(p32, g, m, v, lr, beta1, beta2, eps, weight_decay, step, grad_scale)
        if p_lowp is not None:
            p_lowp.copy_(p32)
        return
    _ext().adamw_step(p32, g, m, v, p_lowp, lr, beta1, beta2, eps, weight_decay, step, grad_scale)
    _count()
