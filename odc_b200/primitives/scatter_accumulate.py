"""``scatter_accumulate``: the producer adds its gradient rows straight into the owners' shards.

Contract of the reference's ``ReductionService`` (odc/primitives/scatter_accumulate.py:494-749):
``input`` is 1-D and rank-major ``[|pg|, shard]``; row p is ADDED into rank p's persistent
accumulator for ``key``; accumulators have ``accumulation_dtype`` (default: the input dtype);
the sum on an owner is complete only after ``sync`` on that owner; ``clear_accumulations``
zeroes them (the caller fences with a barrier); ``get_accumulation`` returns the live tensor.

What differs: there is no mailbox, no request/ack word and no watcher process
(scatter_accumulate.py:267-491).  The producer's kernel issues vector ``red.global.add``
through the peer mapping into the owner's accumulator — each gradient byte crosses NVLink once
and is never staged — and finishes by bumping an arrival counter on every owner with a
system-scope release.  ``sync`` makes the per-owner dispatch counts known to the owners — each producer
stores its count in its slot on the owner (no host collective), or, when a payload rides along, through one host
exchange — and then runs one bounded device wait until the local counter has caught up.  The counter is cumulative
and never reset, so no acknowledgement travels back to the producer and ``input`` may be reused
as soon as the call's kernel has run (stream order).
"""
from __future__ import annotations

import logging
from typing import Dict, Hashable, Optional

import torch
import torch.distributed as dist

from .. import config
from ..runtime import control
from ..runtime.registry import SymmBufferRegistry
from ..runtime.transport import Transport, make_transport
from ..utils.nvtx import nvtx_range

logger = logging.getLogger("odc_b200")

COUNTER_KEY = "odc_arrival_counter"
POSTED_KEY = "odc_posted_counts"


def accumulation_key(key: Hashable) -> str:
    return f"rs_accumulation_{key}"


def slots_key(key: Hashable) -> str:
    return f"rs_slots_{key}"


class ReductionService:
    def __init__(self, accumulation_dtype: Optional[torch.dtype] = None, transport: Optional[Transport] = None):
        self.registry = SymmBufferRegistry.get_instance()
        self.transport = transport or make_transport(self.registry)
        self.accumulation_dtype = accumulation_dtype
        self.accumulations: Dict[Hashable, torch.Tensor] = {}
        self.dispatched: Dict[int, int] = {}   # owner global rank -> contributions sent (cumulative)
        self.expected_total = 0                 # contributions this rank has been told to expect
        # deterministic mode: one slot per producer on every owner, reduced in rank order at sync
        self.deterministic = config.deterministic()
        self.slots: Dict[Hashable, torch.Tensor] = {}
        self.counter = self.registry.get_or_create_symm_buffer(COUNTER_KEY, (8,), torch.int64)
        self.counter.zero_()
        # slot p: what producer p has told this rank about its dispatches (synchronisation number << 32 | count)
        self.posted = self.registry.get_or_create_symm_buffer(POSTED_KEY, (max(8, control.world_size()),), torch.int64)
        self.posted.zero_()
        self.epoch = 0
        control.heartbeat()  # starts publishing (if enabled) before the barrier, so every peer is seen alive after it
        self._sync_device()
        control.host_barrier()
        self.calls = 0

    def _sync_device(self):
        if self.counter.is_cuda:
            torch.cuda.current_stream().synchronize()

    # -- registration (collective) ---------------------------------------------------------
    def register(self, key: Hashable, shard_numel: int, input_dtype: torch.dtype,
                 pg: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
        """Collective over all ranks: allocate and zero the accumulator of ``key``."""
        if key in self.accumulations:
            return self.accumulations[key]
        acc_dtype = self.accumulation_dtype or input_dtype
        acc = self.registry.get_or_create_symm_buffer(accumulation_key(key), (shard_numel,), acc_dtype)
        acc.zero_()
        if self.deterministic:
            slots = self.registry.get_or_create_symm_buffer(slots_key(key), (control.world_size(), shard_numel), acc_dtype)
            slots.zero_()
            self.slots[key] = slots
        self._sync_device()
        control.host_barrier()
        self.accumulations[key] = acc
        return acc

    # -- hot path ----------------------------------------------------------------------------
    def scatter_accumulate(self, key: Hashable, input: torch.Tensor, pg: Optional[dist.ProcessGroup] = None,
                           scale: float = 1.0) -> None:
        ranks = control.group_ranks(pg)
        n = len(ranks)
        if input.dim() != 1:
            input = input.reshape(-1)
        if input.numel() % n != 0:
            raise ValueError(f"input of {input.numel()} elements is not a multiple of the group size {n}")
        shard = input.numel() // n
        acc = self.accumulations.get(key)
        if acc is None:
            acc = self.register(key, shard, input.dtype, pg)  # first call per key is collective
        if acc.numel() != shard:
            raise ValueError(f"accumulator of {key!r} holds {acc.numel()} elements, input rows have {shard}")
        me = control.rank()
        my_index = ranks.index(me)
        target = self.scatter_target(key)
        with nvtx_range("odc::scatter_accumulate"):
            self.transport.scatter_add(input.view(n, shard), target, self.counter, ranks, my_index, scale)
        self.note_dispatch(ranks)

    def scatter_accumulate_segments(self, key: Hashable, grads, chunk_numels, dst_offsets,
                                    pg: Optional[dist.ProcessGroup] = None, scale: float = 1.0) -> bool:
        """One contribution to ``key`` taken straight from a list of contiguous tensors.

        Tensor i is split along dim 0 into ``|pg|`` chunks of ``chunk_numels[i]`` elements (the last owners get
        fewer or none when the tensor is shorter than ``|pg|`` chunks) and chunk r is added at element
        ``dst_offsets[i]`` of rank r's accumulator.  The accumulator must be registered.  Returns False without
        doing anything when the transport cannot do this in place; the caller then builds the rank-major
        input and calls :meth:`scatter_accumulate`.
        """
        ranks = control.group_ranks(pg)
        target = self.scatter_target(key)
        with nvtx_range("odc::scatter_accumulate"):
            done = self.transport.scatter_add_segments(grads, chunk_numels, dst_offsets, target, self.counter, ranks,
                                                       ranks.index(control.rank()), scale)
        if done:
            self.note_dispatch(ranks)
        return done

    def note_dispatch(self, ranks) -> None:
        """Record one contribution sent to each of ``ranks`` (also used by the fused weight-gradient GEMM)."""
        for r in ranks:
            self.dispatched[r] = self.dispatched.get(r, 0) + 1
        self.calls += 1

    def get_accumulation(self, key: Hashable) -> torch.Tensor:
        return self.accumulations[key]

    def scatter_target(self, key: Hashable) -> torch.Tensor:
        """The buffer a producer adds into on every owner: the shared accumulator, or this rank's slot."""
        return self.slots[key][control.rank()] if self.deterministic else self.accumulations[key]

    def has_accumulation(self, key: Hashable) -> bool:
        return key in self.accumulations

    def clear_accumulations(self) -> None:
        for acc in self.accumulations.values():
            acc.zero_()
        for slots in self.slots.values():
            slots.zero_()

    # -- once per minibatch ------------------------------------------------------------------
    def sync(self, pg: Optional[dist.ProcessGroup] = None, payload=None) -> list:
        """Collective over all ranks: wait until every contribution addressed to this rank has landed.

        ``payload`` (any picklable object) rides on the one host exchange this call makes; the list of every
        rank's payload is returned, so callers need no collective of their own at the minibatch boundary.
        """
        with nvtx_range("odc::scatter_accumulate_sync"):
            me = control.rank()
            world = list(range(control.world_size()))
            self.epoch += 1
            control.check_peers_alive()  # host-side liveness first: a rank that left is reported, not waited for
            if payload is None and config.sync_by_posting() and self.transport.supports_posting(world):
                # No host collective: every producer stores its cumulative count on each owner, and the owner's
                # wait collects the postings of this synchronisation before it waits for the arrivals themselves.
                self.transport.post_counts(self.posted, world, me, self.epoch,
                                           [self.dispatched.get(r, 0) for r in world])
                self.transport.wait_posted(self.posted, self.counter, len(world), self.epoch)
                self.expected_total = None  # summed on the device; not brought back to the host
                gathered = [(None, None)] * len(world)
            else:
                gathered = control.all_gather_object((dict(self.dispatched), payload))
                everyone = [d for d, _ in gathered]
                self.expected_total = sum(d.get(me, 0) for d in everyone)
                self.transport.wait_arrivals(self.counter, self.expected_total)
            if self.deterministic:
                for key, slots in self.slots.items():  # fixed order: rank 0 first
                    acc = self.accumulations[key]
                    acc.zero_()
                    for r in range(slots.shape[0]):
                        acc.add_(slots[r])
            return [x for _, x in gathered]

    def stop(self) -> None:
        self._sync_device()
        control.host_barrier()
        self.accumulations.clear()
        self.slots.clear()
