"""Synthetic variable-length workloads and packed microbatches.

Length distributions: ``uniform`` (oracle config), ``lognormal`` (median/sigma/cap) and
``longtail`` (RL-style rollouts: 75 % short, 25 % very long).  Each rank draws its own
sequences from an independently seeded generator, so ranks are deliberately imbalanced.

A microbatch is one packed row (examples/llm_training/data.py:103-127): ``input_ids``,
``position_ids`` restarting per sequence, ``cu_seqlens``, next-token ``labels`` and a per-token
``loss_scale = 1 / len / sequences_in_minibatch`` with the last token of each sequence zeroed.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .packing import CostFn, rearrange_micro_batches


@dataclass
class LengthSpec:
    kind: str = "lognormal"       # uniform | lognormal | longtail | fixed
    lo: int = 16
    hi: int = 128
    median: float = 512.0
    sigma: float = 1.0
    cap: int = 8192
    short: tuple = (256, 2048)
    long: tuple = (8192, 32768)
    long_frac: float = 0.25


def sample_lengths(spec: LengthSpec, n: int, rng: np.random.Generator) -> List[int]:
    if spec.kind == "fixed":
        return [spec.hi] * n
    if spec.kind == "uniform":
        return rng.integers(spec.lo, spec.hi + 1, size=n).tolist()
    if spec.kind == "lognormal":
        x = rng.lognormal(mean=math.log(spec.median), sigma=spec.sigma, size=n)
        return np.clip(np.rint(x), spec.lo, spec.cap).astype(np.int64).tolist()
    if spec.kind == "longtail":
        is_long = rng.random(n) < spec.long_frac
        s = rng.integers(spec.short[0], spec.short[1] + 1, size=n)
        l = rng.integers(spec.long[0], spec.long[1] + 1, size=n)
        return np.where(is_long, l, s).astype(np.int64).tolist()
    raise ValueError(spec.kind)


def sample_until_budget(spec: LengthSpec, token_budget: int, rng: np.random.Generator) -> List[int]:
    """Draw sequences until the next one would exceed ``token_budget`` tokens in total."""
    out, total = [], 0
    while True:
        n = sample_lengths(spec, 1, rng)[0]
        if total + n > token_budget:
            if not out:
                out.append(min(n, token_budget))
            return out
        out.append(n); total += n


def pack_microbatch(seqs: Sequence[torch.Tensor], minibatch_num_seqs: int, pin: bool = False) -> Dict[str, torch.Tensor]:
    lens = [int(s.numel()) for s in seqs]
    ids = torch.cat(list(seqs)).to(torch.int64)
    pos = torch.cat([torch.arange(n, dtype=torch.int64) for n in lens])
    cu = torch.zeros(len(lens) + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(lens, dtype=torch.int32).cumsum(0)
    labels = torch.roll(ids, -1)
    scale = torch.cat([torch.full((n,), 1.0 / n / minibatch_num_seqs, dtype=torch.float32) for n in lens])
    last = cu[1:].long() - 1
    scale[last] = 0.0
    labels[last] = -100
    mb = {"input_ids": ids, "position_ids": pos, "cu_seqlens": cu, "labels": labels, "loss_scale": scale}
    if pin:
        mb = {k: v.pin_memory() for k, v in mb.items()}
    mb["max_seqlen"] = max(lens)
    mb["num_seqs"] = len(lens)
    mb["num_tokens"] = int(ids.numel())
    return mb


def make_minibatch(rank: int, step: int, vocab: int, spec: LengthSpec, microbatches: int, token_budget: int,
                   seed: int = 0, pin: bool = False, pad_to: int = 1) -> List[Dict[str, torch.Tensor]]:
    """``microbatches`` packed rows for one rank, each filled up to ``token_budget`` tokens."""
    rng = np.random.default_rng([seed, rank, step])
    rows = [sample_until_budget(spec, token_budget, rng) for _ in range(microbatches)]
    nseq = sum(len(r) for r in rows)
    out = []
    for lens in rows:
        seqs = [torch.from_numpy(rng.integers(0, vocab, size=n)) for n in lens]
        out.append(pack_microbatch(seqs, nseq, pin))
    return out


def make_minibatch_from_lengths(lengths: Sequence[int], vocab: int, max_token_len: int, seed: int = 0,
                                cost_fn: Optional[CostFn] = None, pin: bool = False):
    """Token-budgeted, cost-balanced microbatches for a given list of this rank's sequence lengths."""
    rng = np.random.default_rng(seed)
    parts = rearrange_micro_batches(list(lengths), max_token_len, cost_fn=cost_fn)
    out = []
    for p in parts:
        seqs = [torch.from_numpy(rng.integers(0, vocab, size=lengths[i])) for i in p]
        out.append(pack_microbatch(seqs, len(lengths), pin))
    return out


def to_device(mb: Dict, device, non_blocking: bool = True) -> Dict:
    return {k: (v.to(device, non_blocking=non_blocking) if torch.is_tensor(v) else v) for k, v in mb.items()}


def h2d_bytes(mb: Dict) -> int:
    return sum(v.numel() * v.element_size() for v in mb.values() if torch.is_tensor(v))
