"""Llama / Qwen2-style decoder on packed variable-length batches.

The reference trains Hugging Face ``Qwen2ForCausalLM`` with flash-attn-2 varlen and a chunked LM
head (examples/llm_training/torch_fsdp2.py:85-106, lm_head.py:7-59).  This decoder has the same
architecture family (RMSNorm, rotary GQA attention, SwiGLU, optional QKV bias, optional tied
embeddings) but is written against :mod:`odc_b200.ops`, so on a GPU every layer runs the
package's sm_100a kernels.  Projections are stored fused (``wqkv``, ``w_gate_up``) so that one
GEMM feeds rotary/attention and one feeds SwiGLU.

Inputs are one packed row per microbatch: ``input_ids [T]``, ``position_ids [T]`` restarting at
each sequence, ``cu_seqlens [S+1]``.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint

from .. import ops


@dataclass
class DecoderConfig:
    vocab_size: int = 1024
    hidden_size: int = 256
    intermediate_size: int = 688
    num_layers: int = 2
    num_heads: int = 4
    num_kv_heads: int = 4
    head_dim: int = 64
    rms_eps: float = 1e-6
    rope_theta: float = 10000.0
    tie_embeddings: bool = False
    qkv_bias: bool = False
    init_std: float = 0.02
    activation_checkpointing: bool = False
    ce_chunk: int = 4096
    # rescaled rotary frequencies ({"rope_type": "llama3" | "linear", "factor": ...}, see ops.reference.rope_inv_freq);
    # None = plain theta^(-2i/d), which is what the rotary kernel computes itself
    rope_scaling: Optional[dict] = None

    def rope_inv_freq(self, device) -> Optional[torch.Tensor]:
        """The rescaled frequencies on ``device`` (cached), or None when the kernel's own frequencies apply."""
        if not self.rope_scaling or self.rope_scaling.get("rope_type", "default") == "default":
            return None
        cache = self.__dict__.setdefault("_inv_freq_cache", {})
        key = str(device)
        if key not in cache:
            from ..ops.reference import rope_inv_freq
            cache[key] = rope_inv_freq(self.head_dim, self.rope_theta, self.rope_scaling, device=device)
        return cache[key]

    @property
    def qkv_dim(self) -> int:
        return (self.num_heads + 2 * self.num_kv_heads) * self.head_dim

    def num_params(self) -> int:
        h, f = self.hidden_size, self.intermediate_size
        per_layer = self.qkv_dim * h + (self.qkv_dim if self.qkv_bias else 0) + h * self.num_heads * self.head_dim \
            + 3 * h * f + 2 * h
        emb = self.vocab_size * h * (1 if self.tie_embeddings else 2)
        return self.num_layers * per_layer + emb + h

    def flops_per_token(self, avg_context: float = 0.0) -> float:
        """Training FLOPs per token: 6 x (matmul parameters) + causal attention at ``avg_context``."""
        h, f = self.hidden_size, self.intermediate_size
        mm = self.num_layers * (self.qkv_dim * h + h * self.num_heads * self.head_dim + 3 * h * f) \
            + self.vocab_size * h
        attn = self.num_layers * 2 * self.num_heads * self.head_dim * avg_context  # qk^T + pv, causal half
        return 6.0 * mm + 3.0 * 2.0 * attn


PRESETS = {
    # plumbing / loss-parity oracle
    "tiny": DecoderConfig(),
    "llama3.2-1b": DecoderConfig(vocab_size=128256, hidden_size=2048, intermediate_size=8192, num_layers=16,
                                 num_heads=32, num_kv_heads=8, head_dim=64, rms_eps=1e-5, rope_theta=500000.0,
                                 tie_embeddings=True),
    "llama3-8b": DecoderConfig(vocab_size=128256, hidden_size=4096, intermediate_size=14336, num_layers=32,
                               num_heads=32, num_kv_heads=8, head_dim=128, rms_eps=1e-5, rope_theta=500000.0),
    "qwen2.5-14b": DecoderConfig(vocab_size=152064, hidden_size=5120, intermediate_size=13824, num_layers=48,
                                 num_heads=40, num_kv_heads=8, head_dim=128, rms_eps=1e-6, rope_theta=1000000.0,
                                 qkv_bias=True),
    "qwen2.5-1.5b": DecoderConfig(vocab_size=151936, hidden_size=1536, intermediate_size=8960, num_layers=28,
                                  num_heads=12, num_kv_heads=2, head_dim=128, rms_eps=1e-6, rope_theta=1000000.0,
                                  qkv_bias=True, tie_embeddings=True),
}


def get_config(name: str, **overrides) -> DecoderConfig:
    return replace(PRESETS[name], **overrides)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return ops.rms_norm(x, self.weight, self.eps)

    def with_residual(self, x):
        """``(norm(x), x)``; backward folds the residual path's gradient into the norm's backward kernel."""
        return ops.rms_norm_residual(x, self.weight, self.eps)


class Attention(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg
        self.wqkv = nn.Parameter(torch.empty(cfg.qkv_dim, cfg.hidden_size))
        self.bqkv = nn.Parameter(torch.zeros(cfg.qkv_dim)) if cfg.qkv_bias else None
        self.wo = nn.Parameter(torch.empty(cfg.hidden_size, cfg.num_heads * cfg.head_dim))

    def forward(self, x, position_ids, cu_seqlens, max_seqlen, residual=None):
        c = self.cfg
        T = x.shape[0]
        qkv = ops.linear(x, self.wqkv, self.bqkv)
        qkv = ops.rope_qkv(qkv, position_ids, c.num_heads, c.num_kv_heads, c.head_dim, c.rope_theta,
                           c.rope_inv_freq(qkv.device))
        nq = c.num_heads * c.head_dim
        o = ops.varlen_attention_qkv(qkv, c.num_heads, c.num_kv_heads, c.head_dim, cu_seqlens, max_seqlen, causal=True)
        return ops.linear(o.reshape(T, nq), self.wo, residual=residual)


class MLP(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.w_gate_up = nn.Parameter(torch.empty(2 * cfg.intermediate_size, cfg.hidden_size))
        self.w_down = nn.Parameter(torch.empty(cfg.hidden_size, cfg.intermediate_size))

    def forward(self, x, residual=None):
        return ops.linear(ops.swiglu(ops.linear(x, self.w_gate_up)), self.w_down, residual=residual)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.attn_norm = RMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.attn = Attention(cfg)
        self.mlp_norm = RMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.mlp = MLP(cfg)

    def forward(self, x, position_ids, cu_seqlens, max_seqlen):
        h, x = self.attn_norm.with_residual(x)
        x = self.attn(h, position_ids, cu_seqlens, max_seqlen, residual=x)
        h, x = self.mlp_norm.with_residual(x)
        return self.mlp(h, residual=x)


class DecoderLM(nn.Module):
    def __init__(self, cfg: DecoderConfig):
        super().__init__()
        self.cfg = cfg
        self.embed = nn.Embedding(cfg.vocab_size, cfg.hidden_size)
        self.layers = nn.ModuleList([DecoderLayer(cfg) for _ in range(cfg.num_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_eps)
        self.lm_head = None if cfg.tie_embeddings else nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size))
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self, seed: Optional[int] = None):
        gen = None
        if seed is not None:
            gen = torch.Generator(device=self.embed.weight.device).manual_seed(seed)
        for name, p in self.named_parameters():
            if p.dim() >= 2:
                p.normal_(0.0, self.cfg.init_std, generator=gen)
            elif name.endswith("weight"):
                p.fill_(1.0)
            else:
                p.zero_()

    def head_weight(self):
        return self.embed.weight if self.lm_head is None else self.lm_head

    def hidden_states(self, input_ids, position_ids, cu_seqlens, max_seqlen):
        x = self.embed(input_ids)
        for layer in self.layers:
            if self.cfg.activation_checkpointing and torch.is_grad_enabled():
                x = checkpoint(layer, x, position_ids, cu_seqlens, max_seqlen, use_reentrant=False)
            else:
                x = layer(x, position_ids, cu_seqlens, max_seqlen)
        return self.norm(x)

    def forward(self, input_ids, position_ids, cu_seqlens, max_seqlen, labels=None, loss_scale=None,
                return_logprobs: bool = False, temperature: float = 1.0):
        """Summed (``loss_scale``-weighted) next-token loss if ``labels`` is given, else final hidden states.

        With ``return_logprobs`` the per-token log-probabilities of ``labels`` come back instead of the loss
        (fp32, 0 at ignored positions): what policy-gradient objectives weight by an advantage, and what the
        reference's trainers build their loss from (examples/llm_training/torch_fsdp2.py:70-80).
        """
        h = self.hidden_states(input_ids, position_ids, cu_seqlens, max_seqlen)
        if labels is None:
            return h
        if return_logprobs:
            return ops.linear_token_logprobs(h, self.head_weight(), labels, temperature, chunk=self.cfg.ce_chunk)
        return ops.linear_cross_entropy(h, self.head_weight(), labels, loss_scale, chunk=self.cfg.ce_chunk)

    def logits(self, input_ids, position_ids, cu_seqlens, max_seqlen):
        return ops.linear(self.hidden_states(input_ids, position_ids, cu_seqlens, max_seqlen), self.head_weight())
