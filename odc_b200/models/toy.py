"""Toy GPT-style Transformer (LayerNorm, scaled-dot-product attention, GELU MLP).

Stands in for the reference's FSDP2 example model (examples/FSDP2/model.py:98-132): dense
``[B, S]`` batches, learned positions, useful for quick FSDP2/HSDP/HPZ plumbing checks.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class ToyConfig:
    vocab_size: int = 1024
    max_seq_len: int = 64
    dim: int = 128
    n_layers: int = 2
    n_heads: int = 4
    dropout: float = 0.0


class ToyBlock(nn.Module):
    def __init__(self, c: ToyConfig):
        super().__init__()
        self.n_heads = c.n_heads
        self.ln1, self.ln2 = nn.LayerNorm(c.dim), nn.LayerNorm(c.dim)
        self.qkv = nn.Linear(c.dim, 3 * c.dim)
        self.proj = nn.Linear(c.dim, c.dim)
        self.fc1, self.fc2 = nn.Linear(c.dim, 4 * c.dim), nn.Linear(4 * c.dim, c.dim)

    def forward(self, x):
        B, S, D = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, S, 3, self.n_heads, D // self.n_heads).permute(2, 0, 3, 1, 4)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, S, D)
        x = x + self.proj(a)
        return x + self.fc2(F.gelu(self.fc1(self.ln2(x))))


class ToyTransformer(nn.Module):
    def __init__(self, c: ToyConfig):
        super().__init__()
        self.tok = nn.Embedding(c.vocab_size, c.dim)
        self.pos = nn.Embedding(c.max_seq_len, c.dim)
        self.layers = nn.ModuleList([ToyBlock(c) for _ in range(c.n_layers)])
        self.norm = nn.LayerNorm(c.dim)
        self.out = nn.Linear(c.dim, c.vocab_size, bias=False)

    def forward(self, tokens):
        S = tokens.shape[1]
        x = self.tok(tokens) + self.pos(torch.arange(S, device=tokens.device))
        for layer in self.layers:
            x = layer(x)
        return self.out(self.norm(x))
