"""Global batch -> per-rank packed microbatches (examples/llm_training/data.py:6-100)."""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch

from .packing import get_packing_function
from .synthetic import pack_microbatch


class BatchedDataset:
    """Indexes a list of token sequences by global batch; returns this rank's microbatches.

    ``sequences`` is anything indexable that yields 1-D integer tensors (or lists).  Sequences
    longer than ``limit_token_len`` are dropped (or truncated if none fits), and the batch is
    padded by repetition to a multiple of the world size, as equal-count strategies need.
    """

    def __init__(self, sequences: Sequence, batch_size: int, rank: int, world_size: int,
                 packing_method: str = "None", max_token_len: int = 65536, limit_token_len: Optional[int] = None,
                 cost_fn=None, odc_enabled: bool = True):
        self.sequences, self.batch_size, self.rank, self.world_size = sequences, batch_size, rank, world_size
        self.global_batch = batch_size * world_size
        self.limit = limit_token_len
        self.pack = get_packing_function(packing_method, max_token_len, cost_fn, odc_enabled)
        self.last_debug = ""

    def __len__(self):
        return len(self.sequences) // self.global_batch

    def __getitem__(self, index) -> List[Dict[str, torch.Tensor]]:
        idx = range(index * self.global_batch, (index + 1) * self.global_batch)
        seqs = [torch.as_tensor(self.sequences[i]) for i in idx]
        if self.limit is not None:
            keep = [s for s in seqs if s.numel() <= self.limit]
            seqs = keep if keep else [s[: self.limit] for s in seqs]
            n = len(seqs)
            for i in range((-n) % self.world_size):
                seqs.append(seqs[i % n].clone())
        lengths = [int(s.numel()) for s in seqs]
        groups = self.pack(lengths, self.rank, self.world_size)
        self.last_debug = f"rank {self.rank} " + "; ".join(
            "+".join(str(lengths[i]) for i in g) + f"={sum(lengths[i] for i in g)}" for g in groups)
        return [pack_microbatch([seqs[i] for i in g], self.batch_size) for g in groups if g]
