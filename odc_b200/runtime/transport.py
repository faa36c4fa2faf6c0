"""Transports: how bytes reach a peer's region of the symmetric heap.

The primitives talk to this small interface, so the data plane can be swapped without
touching the FSDP integration:

* :class:`NvlinkP2PTransport` — same-node GPUs.  One kernel launch per call; CTAs issue
  16-byte peer loads (gather) or vector ``red.global.add`` (scatter-accumulate) through the
  heap's peer mappings over NVLink/NVSwitch, and bump the owners' arrival counters with a
  system-scope release.
* :class:`HostShmTransport` — CPU ranks over the ``/dev/shm`` heap; the functional model used
  by the CPU/gloo tests.
* :class:`InterNodeTransport` — ranks of other nodes (the reference's NVSHMEM get/put kernels,
  odc/primitives/gather.py:22-64 and scatter_accumulate.py:42-174): one-sided get / add by heap
  offset, served by a small TCP server on every rank and staged through host memory.
* :class:`HybridTransport` — splits a group into same-node and other-node members and uses the two
  above; what the services get when the job spans more than one node.
"""
from __future__ import annotations

import time
from typing import Sequence

import torch

from .. import config
from .heap import HostShmHeap, SymmetricHeap
from .registry import SymmBufferRegistry
from .status import OdcTimeoutError, check_status_word


class Transport:
    def gather(self, out2d: torch.Tensor, src_local: torch.Tensor, ranks: Sequence[int], my_index: int) -> None:
        """``out2d[i] <- (buffer `src_local` on rank ranks[i])`` for every i, converting dtype."""
        raise NotImplementedError

    def scatter_add(self, inp2d: torch.Tensor, acc_local: torch.Tensor, counter_local: torch.Tensor,
                    ranks: Sequence[int], my_index: int, scale: float = 1.0) -> None:
        """``acc on ranks[i] += scale * inp2d[i]``, then one arrival on each owner's counter."""
        raise NotImplementedError

    def wait_arrivals(self, counter_local: torch.Tensor, expected: int) -> None:
        """Return once the local arrival counter has reached ``expected`` (bounded)."""
        raise NotImplementedError

    def scatter_add_segments(self, grads, chunk_numels, dst_offsets, acc_local: torch.Tensor,
                             counter_local: torch.Tensor, ranks: Sequence[int], my_index: int,
                             scale: float = 1.0) -> bool:
        """``scatter_add`` taken straight from a list of contiguous tensors (no flattened staging copy).

        Tensor i is split along dim 0 into chunks of ``chunk_numels[i]`` elements, chunk r is added at element
        ``dst_offsets[i]`` of the accumulator on ``ranks[r]``; one arrival per owner.  Returns False, having done
        nothing, when this transport has no such path: the caller then flattens and calls ``scatter_add``.
        """
        return False

    # -- one-sided exchange of dispatch counts (``sync`` without a host collective) --------------------------------
    def supports_posting(self, ranks: Sequence[int]) -> bool:
        """True when this transport can store a word directly on every one of ``ranks``."""
        return False

    def post_counts(self, slots_local: torch.Tensor, ranks: Sequence[int], my_slot: int, epoch: int,
                    counts: Sequence[int]) -> None:
        """Store ``(epoch << 32) | counts[i]`` in slot ``my_slot`` of buffer ``slots_local`` on ``ranks[i]``."""
        raise NotImplementedError

    def wait_posted(self, slots_local: torch.Tensor, counter_local: torch.Tensor, nprod: int, epoch: int) -> None:
        """Collect one posting of ``epoch`` from each of ``nprod`` producers, then wait for that many arrivals."""
        raise NotImplementedError


class HostShmTransport(Transport):
    def __init__(self, registry: SymmBufferRegistry):
        assert isinstance(registry.heap, HostShmHeap)
        self.registry = registry
        self.heap: HostShmHeap = registry.heap

    def gather(self, out2d, src_local, ranks, my_index):
        peers = self.registry.get_peer_tensors(src_local)
        n = len(ranks)
        for k in range(n):
            i = (my_index + k) % n  # own shard first, rotated start (gather.py:121-122)
            out2d[i].copy_(peers[ranks[i]].view(-1))

    def scatter_add(self, inp2d, acc_local, counter_local, ranks, my_index, scale=1.0):
        accs = self.registry.get_peer_tensors(acc_local)
        ctrs = self.registry.get_peer_tensors(counter_local)
        n = len(ranks)
        for k in range(n):
            i = (my_index + k) % n
            r = ranks[i]
            src = inp2d[i].to(accs[r].dtype)
            with self.heap.owner_lock(r):
                if scale != 1.0:
                    accs[r].view(-1).add_(src, alpha=scale)
                else:
                    accs[r].view(-1).add_(src)
                ctrs[r][0] += 1

    def scatter_add_segments(self, grads, chunk_numels, dst_offsets, acc_local, counter_local, ranks, my_index,
                             scale=1.0):
        accs = self.registry.get_peer_tensors(acc_local)
        ctrs = self.registry.get_peer_tensors(counter_local)
        n = len(ranks)
        for k in range(n):
            i = (my_index + k) % n
            r = ranks[i]
            with self.heap.owner_lock(r):
                acc = accs[r].view(-1)
                for g, chunk, off in zip(grads, chunk_numels, dst_offsets):
                    flat = g.reshape(-1)
                    piece = flat[i * chunk:min((i + 1) * chunk, flat.numel())]  # short or empty past the end
                    if piece.numel():
                        acc[off:off + piece.numel()].add_(piece.to(acc.dtype), alpha=scale)
                ctrs[r][0] += 1
        return True

    def wait_arrivals(self, counter_local, expected):
        deadline = time.monotonic() + config.wait_timeout_ms() / 1e3
        while int(counter_local[0]) < expected:
            if time.monotonic() > deadline:
                raise OdcTimeoutError(
                    f"rank {self.heap.rank}: {int(counter_local[0])} of {expected} gradient contributions "
                    f"arrived within {config.wait_timeout_ms()} ms")
            time.sleep(0.0002)

    def supports_posting(self, ranks):
        return all(self.heap.is_local(r) for r in ranks)

    def post_counts(self, slots_local, ranks, my_slot, epoch, counts):
        slots = self.registry.get_peer_tensors(slots_local)
        for r, c in zip(ranks, counts):
            with self.heap.owner_lock(r):
                slots[r][my_slot] = (int(epoch) << 32) | int(c)

    def wait_posted(self, slots_local, counter_local, nprod, epoch):
        deadline = time.monotonic() + config.wait_timeout_ms() / 1e3
        while True:
            words = [int(v) for v in slots_local[:nprod]]
            if all((w >> 32) >= epoch for w in words):
                break
            if time.monotonic() > deadline:
                late = [p for p, w in enumerate(words) if (w >> 32) < epoch]
                raise OdcTimeoutError(f"rank {self.heap.rank}: producers {late} did not post their dispatch counts "
                                      f"for synchronisation {epoch} within {config.wait_timeout_ms()} ms")
            time.sleep(0.0002)
        self.wait_arrivals(counter_local, sum(w & 0xFFFFFFFF for w in words))


class NvlinkP2PTransport(Transport):
    def __init__(self, registry: SymmBufferRegistry):
        from .. import _ext

        self.ext = _ext.load()
        self.registry = registry
        self.heap: SymmetricHeap = registry.heap
        # [0] error code, [1] detail, [2] observed value, [3] spare — written by kernels that give up.  ONE word per
        # device, shared with the GEMM, attention and fused compute+communication kernels, so that the copy `check`
        # makes at every synchronisation point also sees a pipeline wait that ran out inside one of those.
        with torch.cuda.device(self.heap.device):
            self.status = self.ext.kernel_status()
        self._status_host = torch.zeros(4, dtype=torch.int32).pin_memory()
        self._expected = None
        self.launches = 0

    def gather(self, out2d, src_local, ranks, my_index):
        table = self.registry.peer_ptr_table(src_local, ranks)
        self.ext.gather(out2d, table, out2d.shape[1], src_local.dtype, my_index, config.debug_bounds(),
                        self.status, src_local.numel())
        self.launches += 1

    def scatter_add(self, inp2d, acc_local, counter_local, ranks, my_index, scale=1.0):
        acc_table = self.registry.peer_ptr_table(acc_local, ranks)
        ctr_table = self.registry.peer_ptr_table(counter_local, ranks)
        self.ext.scatter_accumulate(inp2d, acc_table, ctr_table, inp2d.shape[1], acc_local.dtype,
                                    my_index, float(scale), config.debug_bounds(), self.status, acc_local.numel())
        self.launches += 1

    def scatter_add_segments(self, grads, chunk_numels, dst_offsets, acc_local, counter_local, ranks, my_index,
                             scale=1.0):
        acc_table = self.registry.peer_ptr_table(acc_local, ranks)
        ctr_table = self.registry.peer_ptr_table(counter_local, ranks)
        done = self.ext.scatter_accumulate_segments(list(grads), [int(c) for c in chunk_numels],
                                                    [int(o) for o in dst_offsets], acc_table, ctr_table,
                                                    acc_local.dtype, my_index, float(scale), config.debug_bounds(),
                                                    self.status, acc_local.numel())
        if done:
            self.launches += 1
        return bool(done)

    def wait_arrivals(self, counter_local, expected):
        self.ext.wait_counter(counter_local, int(expected), config.wait_timeout_ms(), self.status)
        self.launches += 1
        self.check()

    def supports_posting(self, ranks):
        return len(ranks) <= 72 and all(self.heap.is_local(r) for r in ranks)

    def post_counts(self, slots_local, ranks, my_slot, epoch, counts):
        addrs = [a + 8 * my_slot for a in self.registry.peer_ptrs(slots_local, ranks)]
        self.ext.post_counts(addrs, [int(c) for c in counts], int(epoch), self.heap.device.index or 0)
        self.launches += 1

    def wait_posted(self, slots_local, counter_local, nprod, epoch):
        if self._expected is None:
            self._expected = torch.zeros(1, dtype=torch.int64, device=self.heap.device)
        self.ext.wait_posted(slots_local, int(nprod), int(epoch), counter_local, config.wait_timeout_ms(), self.status,
                             self._expected)
        self.launches += 1
        self.check()

    def check(self) -> None:
        """Read the device status word (one small D2H copy + stream sync) and raise if a kernel gave up.

        The word is shared by every kernel of this package on the device, so a GEMM / attention pipeline wait that
        ran out since the last check surfaces here too, at the latest at the next synchronisation point.
        """
        self._status_host.copy_(self.status, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        code = int(self._status_host[0])
        if code != 0:
            detail, seen = int(self._status_host[1]), int(self._status_host[2])
            self.status.zero_()
            check_status_word(code, detail, seen)


class InterNodeTransport(Transport):
    """Ranks of other nodes: one-sided get / add by heap offset through :mod:`odc_b200.runtime.internode`.

    Takes the place of the reference's NVSHMEM get/put kernels (odc/primitives/gather.py:22-64,
    odc/primitives/scatter_accumulate.py:42-174).  Bytes are staged through host memory (pinned on GPU
    jobs) and travel over TCP; the owner's trainer takes no part.
    """

    def __init__(self, registry: SymmBufferRegistry):
        if registry.internode is None:
            raise RuntimeError("the inter-node endpoint was not started (single-node job?)")
        self.registry = registry
        self.endpoint = registry.internode
        self.launches = 0

    def _pieces(self, numel: int, n_peers: int):
        """``(start, length)`` pieces so that one round of requests stages at most ``ODC_MAX_BUFFER_SIZE`` elements."""
        from ..primitives.splitter import BufferSplitter
        splitter = BufferSplitter()
        if splitter.enabled and splitter.max_buffer_size % max(1, n_peers) != 0:
            # the staging cap need not divide by this group's size: use the largest multiple that fits
            splitter = BufferSplitter(max(n_peers, splitter.max_buffer_size // n_peers * n_peers))
        return list(splitter.segments(numel, max(1, n_peers))) or [(0, 0)]

    def gather(self, out2d, src_local, ranks, my_index):
        off = self.registry.offset_of(src_local)
        esz = src_local.element_size()
        for start, length in self._pieces(src_local.numel(), len(ranks)):
            got = self.endpoint.get_many(ranks, off + start * esz, length, src_local.dtype)
            for i, t in enumerate(got):
                out2d[i, start:start + length].copy_(t.view(-1), non_blocking=True)  # converts dtype if they differ
            if out2d.is_cuda:
                torch.cuda.current_stream().synchronize()  # the pinned buffers are released on return

    def scatter_add(self, inp2d, acc_local, counter_local, ranks, my_index, scale=1.0):
        acc_off = self.registry.offset_of(acc_local)
        ctr_off = self.registry.offset_of(counter_local)
        esz = acc_local.element_size()
        pieces = self._pieces(inp2d.shape[1], len(ranks))
        for k, (start, length) in enumerate(pieces):
            part = inp2d[:, start:start + length].detach()
            rows = part.to("cpu") if part.is_cuda else part  # waits for the producing stream
            last = k == len(pieces) - 1
            self.endpoint.add_many(ranks, [rows[i] for i in range(len(ranks))], acc_off + start * esz,
                                   acc_local.dtype, ctr_off if last else -1, scale)

    def wait_arrivals(self, counter_local, expected):
        raise RuntimeError("arrivals are counted on the local counter: wait through the same-node transport")


class HybridTransport(Transport):
    """Same-node ranks over the mapped heap, other nodes through :class:`InterNodeTransport`."""

    def __init__(self, registry: SymmBufferRegistry, intra: Transport, inter: Transport):
        self.registry, self.intra, self.inter = registry, intra, inter
        self.heap = registry.heap
        self._poll_stream = None
        self._poll_host = None

    @property
    def launches(self) -> int:
        return getattr(self.intra, "launches", 0)

    def _runs(self, ranks):
        """Maximal runs ``(start, stop, local?)`` of consecutive group indices on / off this node."""
        runs, a = [], 0
        for i in range(1, len(ranks) + 1):
            if i == len(ranks) or self.heap.is_local(ranks[i]) != self.heap.is_local(ranks[a]):
                runs.append((a, i, self.heap.is_local(ranks[a])))
                a = i
        return runs

    def gather(self, out2d, src_local, ranks, my_index):
        for a, b, local in self._runs(ranks):
            idx = my_index - a if a <= my_index < b else 0
            (self.intra if local else self.inter).gather(out2d[a:b], src_local, ranks[a:b], idx)

    def scatter_add(self, inp2d, acc_local, counter_local, ranks, my_index, scale=1.0):
        for a, b, local in self._runs(ranks):
            idx = my_index - a if a <= my_index < b else 0
            (self.intra if local else self.inter).scatter_add(inp2d[a:b], acc_local, counter_local, ranks[a:b], idx,
                                                              scale)

    def scatter_add_segments(self, grads, chunk_numels, dst_offsets, acc_local, counter_local, ranks, my_index,
                             scale=1.0):
        if any(not self.heap.is_local(r) for r in ranks):
            return False
        return self.intra.scatter_add_segments(grads, chunk_numels, dst_offsets, acc_local, counter_local, ranks,
                                               my_index, scale)

    def wait_arrivals(self, counter_local, expected):
        if not counter_local.is_cuda:
            self.intra.wait_arrivals(counter_local, expected)
            return
        # Contributions from other nodes are added by kernels that this process's own server threads launch.
        # A spinning wait kernel and those kernels would be launches of one GPU that depend on each other, which
        # nothing guarantees to run side by side, so the counter is polled from the host until it is reached.
        if self._poll_stream is None:
            self._poll_stream = torch.cuda.Stream(device=counter_local.device)
            self._poll_host = torch.zeros(1, dtype=torch.int64).pin_memory()
        deadline = time.monotonic() + config.wait_timeout_ms() / 1e3
        while True:
            with torch.cuda.stream(self._poll_stream):
                self._poll_host.copy_(counter_local[:1], non_blocking=True)
            self._poll_stream.synchronize()
            seen = int(self._poll_host[0])
            if seen >= expected:
                break
            if time.monotonic() > deadline:
                raise OdcTimeoutError(f"rank {self.heap.rank}: {seen} of {expected} gradient contributions arrived "
                                      f"within {config.wait_timeout_ms()} ms")
            time.sleep(0.0002)
        self.check()

    def check(self) -> None:
        if hasattr(self.intra, "check"):
            self.intra.check()


def make_transport(registry: SymmBufferRegistry) -> Transport:
    intra = NvlinkP2PTransport(registry) if registry.heap.device.type == "cuda" else HostShmTransport(registry)
    if registry.internode is not None:
        return HybridTransport(registry, intra, InterNodeTransport(registry))
    return intra
