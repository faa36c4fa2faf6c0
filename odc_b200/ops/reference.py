"""Plain PyTorch statements of every op.

These are the CPU implementations (autograd differentiates them) and the fp32 oracles that the
CUDA kernels are tested against.  Shapes use packed variable-length layout: ``T`` tokens of all
sequences of a microbatch concatenated, ``cu_seqlens`` giving sequence boundaries.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def linear(x, w, bias=None):
    return F.linear(x, w, bias)


def rms_norm(x, weight, eps: float):
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return (xf * rstd * weight.float()).to(x.dtype)


def layer_norm(x, weight, bias, eps: float):
    return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(),
                        eps).to(x.dtype)


def rope_inv_freq(head_dim: int, theta: float, scaling: Optional[dict] = None, device=None) -> torch.Tensor:
    """Rotary frequencies ``theta^(-2i/d)``, optionally rescaled.

    ``scaling``: ``{"rope_type": "linear", "factor": f}`` divides every frequency by ``f``;
    ``{"rope_type": "llama3", "factor", "low_freq_factor", "high_freq_factor",
    "original_max_position_embeddings"}`` is the Llama 3.1 / 3.2 rule: components whose wavelength is longer than
    ``original / low_freq_factor`` are slowed down by ``factor``, those shorter than ``original / high_freq_factor``
    are kept, and the band in between is interpolated linearly in ``original / wavelength``.
    """
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    if not scaling or scaling.get("rope_type", "default") == "default":
        return inv
    kind, factor = scaling["rope_type"], float(scaling["factor"])
    if kind == "linear":
        return inv / factor
    if kind != "llama3":
        raise NotImplementedError(f"rotary scaling {kind!r}")
    lo, hi = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    turns = orig * inv / (2.0 * math.pi)                 # rotations completed over the original context
    blend = ((turns - lo) / (hi - lo)).clamp(0.0, 1.0)   # 0: long wavelengths (slowed), 1: short ones (kept)
    return inv * (blend + (1.0 - blend) / factor)


def rope_tables(position_ids: torch.Tensor, head_dim: int, theta: float, inv_freq: Optional[torch.Tensor] = None):
    inv = inv_freq if inv_freq is not None else rope_inv_freq(head_dim, theta, device=position_ids.device)
    ang = position_ids.float()[:, None] * inv.to(position_ids.device)[None, :]
    return ang.cos(), ang.sin()


def rope(x: torch.Tensor, position_ids: torch.Tensor, theta: float, inverse: bool = False,
         inv_freq: Optional[torch.Tensor] = None):
    """Rotate-half rotary embedding on ``x`` of shape ``[T, H, D]`` (HF Llama/Qwen convention)."""
    d = x.shape[-1]
    cos, sin = rope_tables(position_ids, d, theta, inv_freq)
    if inverse:
        sin = -sin
    xf = x.float()
    x1, x2 = xf[..., : d // 2], xf[..., d // 2:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


def swiglu(gate_up: torch.Tensor):
    """``silu(gate) * up`` with ``gate_up = [gate | up]`` along the last dim."""
    f = gate_up.shape[-1] // 2
    g, u = gate_up[..., :f].float(), gate_up[..., f:].float()
    return (F.silu(g) * u).to(gate_up.dtype)


def gelu(x):
    return F.gelu(x)


def varlen_attention(q, k, v, cu_seqlens, causal: bool = True, scale: Optional[float] = None):
    """Attention over packed sequences.  ``q``: [T, Hq, D]; ``k``/``v``: [T, Hkv, D] (GQA)."""
    T, hq, d = q.shape
    hkv = k.shape[1]
    rep = hq // hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    out = torch.empty_like(q)
    bounds = cu_seqlens.tolist()
    for s, e in zip(bounds[:-1], bounds[1:]):
        if e == s:
            continue
        qs = q[s:e].float().transpose(0, 1)                       # [Hq, L, D]
        ks = k[s:e].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vs = v[s:e].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        att = (qs @ ks.transpose(1, 2)) * scale
        if causal:
            L = e - s
            mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
            att = att.masked_fill(~mask, float("-inf"))
        out[s:e] = (att.softmax(-1) @ vs).transpose(0, 1).to(q.dtype)
    return out


def linear_cross_entropy(h, w, labels, loss_scale=None, ignore_index: int = -100, chunk: int = 4096):
    """``sum_t loss_scale[t] * CE(h[t] @ w.T, labels[t])`` without keeping ``[T, vocab]`` logits alive."""
    total = h.new_zeros((), dtype=torch.float32)
    for s in range(0, h.shape[0], chunk):
        logits = F.linear(h[s:s + chunk], w).float()
        lab = labels[s:s + chunk]
        per_tok = F.cross_entropy(logits, lab, reduction="none", ignore_index=ignore_index)
        if loss_scale is not None:
            per_tok = per_tok * loss_scale[s:s + chunk].float()
        total = total + per_tok.sum()
    return total


def linear_token_logprobs(h, w, ids, temperature: float = 1.0, ignore_index: int = -100, chunk: int = 4096):
    """``log_softmax(h @ w.T / temperature)[t, ids[t]]`` per token (0 where ``ids == ignore_index``)."""
    out = []
    for s in range(0, h.shape[0], chunk):
        logits = (F.linear(h[s:s + chunk], w) / temperature).float()
        tok = ids[s:s + chunk]
        keep = tok != ignore_index
        lp = logits.log_softmax(-1).gather(-1, tok.clamp_min(0).unsqueeze(-1)).squeeze(-1)
        out.append(torch.where(keep, lp, torch.zeros_like(lp)))
    return torch.cat(out) if out else h.new_zeros(0, dtype=torch.float32)


def adamw_step(p, g, m, v, lr, beta1, beta2, eps, weight_decay, step, grad_scale: float = 1.0):
    """In-place decoupled-weight-decay Adam on fp32 tensors (matches ``torch.optim.AdamW``)."""
    g = g.float() * grad_scale
    p.mul_(1 - lr * weight_decay)
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    bc1 = 1 - beta1 ** step
    bc2 = 1 - beta2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)
