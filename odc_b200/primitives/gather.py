"""``gather``: the consumer pulls every owner's shard on demand, with no rendezvous.

Contract of the reference's ``GatherService.gather_into_tensor`` (odc/primitives/gather.py:76-176):
``input`` is this rank's registered symmetric shard, ``output`` is rank-major
(``output.view(|pg|, -1)[r]`` is rank r's shard) and the call is ordered after work already
queued on the caller's current stream.  No peer process, stream or kernel takes part, so the
shards must not change while they may be gathered (the barrier in ``pre_minibatch_start``
guarantees that).

What differs: one kernel launch reads all peers (CTAs striped over peers, own shard first), it
can convert dtype while copying (``output.dtype`` may differ from ``input.dtype``, so a bf16
compute copy is produced without a second pass), and the group may be any subset of the ranks
that share the heap (not only WORLD or one node).
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..runtime import control
from ..runtime.registry import SymmBufferRegistry
from ..runtime.transport import Transport, make_transport
from ..utils.nvtx import nvtx_range


class GatherService:
    def __init__(self, transport: Optional[Transport] = None):
        self.registry = SymmBufferRegistry.get_instance()
        self.transport = transport or make_transport(self.registry)
        self.calls = 0

    def gather_into_tensor(self, output: torch.Tensor, input: torch.Tensor,
                           pg: Optional[dist.ProcessGroup] = None, *, use_comm_stream: bool = False) -> None:
        ranks = control.group_ranks(pg)
        if control.rank() not in ranks:
            raise ValueError(f"rank {control.rank()} is not a member of the group {ranks}")
        self.gather_ranks(output, input, ranks, use_comm_stream=use_comm_stream)

    def gather_ranks(self, output: torch.Tensor, input: torch.Tensor, ranks, *,
                     use_comm_stream: bool = False) -> None:
        """Pull buffer ``input`` from an explicit list of global ranks (this rank need not be one of them)."""
        ranks = list(ranks)
        n = len(ranks)
        me = control.rank()
        if output.numel() != input.numel() * n:
            raise ValueError(f"output has {output.numel()} elements, expected {input.numel()} x {n}")
        if not output.is_contiguous():
            raise ValueError("output must be contiguous")
        if self.registry.heap.offset_of(input) is None:
            raise ValueError("input must be a tensor in the symmetric heap (see SymmBufferRegistry)")
        my_index = ranks.index(me) if me in ranks else me % n
        out2d = output.view(n, -1)
        with nvtx_range("odc::gather"):
            stream = control.get_comm_stream() if (use_comm_stream and output.is_cuda) else None
            if stream is not None:
                cur = torch.cuda.current_stream()
                stream.wait_stream(cur)
                with torch.cuda.stream(stream):
                    self.transport.gather(out2d, input, ranks, my_index)
                cur.wait_stream(stream)
            else:
                self.transport.gather(out2d, input, ranks, my_index)
        self.calls += 1
