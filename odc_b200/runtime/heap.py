"""Symmetric heap: one region per rank, every same-node peer's region mapped into every rank.

Takes the place of the NVSHMEM symmetric heap plus ``nvshmem.core.get_peer_tensor``
(odc/primitives/utils.py:54-81) and of the CUDA-IPC helper extension
(csrc/tensor_ipc/tensor_ipc.cu:24-57).  Two implementations share one interface:

* :class:`CudaHeap` — native (``csrc/heap/symm_heap.cpp``): a virtual-address window per
  peer, physical memory created with the CUDA virtual-memory API, exported as POSIX file
  descriptors, passed between ranks over unix sockets and mapped at the same offset in the
  peer's window.  ``ODC_HEAP_MODE=ipc`` selects a ``cudaMalloc`` slab shared through legacy
  CUDA-IPC handles instead.
* :class:`HostShmHeap` — CPU ranks on one host map each other's ``/dev/shm`` files.  It gives
  the CPU/gloo tests true one-sided semantics (a peer's process takes no part in a transfer).

Allocation is collective and deterministic, so an allocation has the same offset on every
rank and ``peer_base[r] + offset`` is the peer's copy of the buffer.
"""
from __future__ import annotations

import fcntl
import logging
import os
import threading
from typing import Dict, List, Optional, Tuple

import torch

from .. import config
from . import control

logger = logging.getLogger("odc_b200")

ALIGN = 512


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


class OffsetAllocator:
    """First-fit free-list allocator over ``[0, capacity)``; pure function of the call sequence."""

    def __init__(self, capacity: int):
        self.capacity = capacity
        self.free: List[Tuple[int, int]] = [(0, capacity)]  # (offset, size), sorted by offset
        self.used: Dict[int, int] = {}

    def alloc(self, nbytes: int) -> int:
        need = _round_up(max(nbytes, 1), ALIGN)
        for i, (off, size) in enumerate(self.free):
            if size >= need:
                if size == need:
                    self.free.pop(i)
                else:
                    self.free[i] = (off + need, size - need)
                self.used[off] = need
                return off
        raise MemoryError(
            f"symmetric heap exhausted: need {need} bytes, capacity {self.capacity}; "
            "raise ODC_SYMMETRIC_SIZE"
        )

    def release(self, off: int) -> None:
        size = self.used.pop(off)
        self.free.append((off, size))
        self.free.sort()
        merged: List[Tuple[int, int]] = []
        for o, s in self.free:
            if merged and merged[-1][0] + merged[-1][1] == o:
                merged[-1] = (merged[-1][0], merged[-1][1] + s)
            else:
                merged.append((o, s))
        self.free = merged

    @property
    def high_water(self) -> int:
        return max((o + s for o, s in self.used.items()), default=0)

    @property
    def bytes_in_use(self) -> int:
        return sum(self.used.values())


class SymmetricHeap:
    """Interface shared by the CUDA and host-shm heaps."""

    device: torch.device
    rank: int
    world: int

    def alloc(self, nbytes: int) -> int:  # collective
        raise NotImplementedError

    def free(self, offset: int) -> None:  # collective
        raise NotImplementedError

    def local(self, offset: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        raise NotImplementedError

    def peer(self, r: int, offset: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        raise NotImplementedError

    def peer_ptr(self, r: int, offset: int) -> int:
        raise NotImplementedError

    def offset_of(self, tensor: torch.Tensor) -> Optional[int]:
        raise NotImplementedError

    def close(self) -> None:
        raise NotImplementedError

    # Only the ranks of this node are mapped; the regions of other nodes are reached through the
    # inter-node transport by heap offset (offsets are the same on every rank).
    node: List[int]

    def is_local(self, r: int) -> bool:
        return self.node[0] <= r <= self.node[-1]

    def _check_local(self, r: int) -> None:
        if not self.is_local(r):
            raise ValueError(f"rank {r} is on another node: its heap region is not mapped on rank {self.rank} "
                             f"(node ranks {self.node[0]}..{self.node[-1]})")


class HostShmHeap(SymmetricHeap):
    """CPU symmetric heap over ``/dev/shm`` files, one per rank."""

    def __init__(self, nbytes: Optional[int] = None):
        self.device = torch.device("cpu")
        self.rank, self.world = control.rank(), control.world_size()
        self.node = control.node_ranks()
        self.nbytes = _round_up(nbytes or config.symmetric_size("cpu"), 4096)
        token = control.job_token()
        self._paths = {r: f"/dev/shm/odc_b200_{token}_{r}" for r in self.node}
        # create mine (sparse), then map the node's after a barrier
        with open(self._paths[self.rank], "wb") as f:
            f.truncate(self.nbytes)
        control.host_barrier()
        self._maps = {
            r: torch.from_file(p, shared=True, size=self.nbytes, dtype=torch.uint8) for r, p in self._paths.items()
        }
        self._lock_fds = {r: os.open(p, os.O_RDWR) for r, p in self._paths.items()}
        self._mutexes = {r: threading.Lock() for r in self._paths}
        self._alloc = OffsetAllocator(self.nbytes)
        self._base = self._maps[self.rank].data_ptr()
        control.host_barrier()
        # every rank of the node has mapped and opened the files: drop the names now, so that nothing is left in
        # /dev/shm however the job ends (mappings and descriptors keep the memory alive)
        try:
            os.unlink(self._paths[self.rank])
        except FileNotFoundError:
            pass

    def alloc(self, nbytes: int) -> int:
        return self._alloc.alloc(nbytes)

    def free(self, offset: int) -> None:
        self._alloc.release(offset)

    def _view(self, r: int, offset: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        nb = numel * torch.empty((), dtype=dtype).element_size()
        if offset < 0 or offset + nb > self.nbytes:
            raise IndexError(f"heap view [{offset}, {offset + nb}) outside region of {self.nbytes} bytes")
        self._check_local(r)
        return self._maps[r][offset : offset + nb].view(dtype)

    def local(self, offset, numel, dtype):
        return self._view(self.rank, offset, numel, dtype)

    def peer(self, r, offset, numel, dtype):
        return self._view(r, offset, numel, dtype)

    def peer_ptr(self, r, offset):
        self._check_local(r)
        return self._maps[r].data_ptr() + offset

    def offset_of(self, tensor):
        p = tensor.data_ptr()
        if self._base <= p < self._base + self.nbytes:
            return p - self._base
        return None

    class _Locked:
        """File lock between processes plus a mutex between the threads of this process.

        ``flock`` belongs to the open file description, so two threads that share the descriptor (the trainer and
        the inter-node server threads of one rank) would both "hold" it; the mutex is what keeps them apart.
        """

        def __init__(self, fd, mutex):
            self.fd, self.mutex = fd, mutex

        def __enter__(self):
            self.mutex.acquire()
            fcntl.flock(self.fd, fcntl.LOCK_EX)

        def __exit__(self, *exc):
            fcntl.flock(self.fd, fcntl.LOCK_UN)
            self.mutex.release()

    def owner_lock(self, r: int):
        """Exclusive lock of rank ``r``'s region: makes a read-modify-write by one producer atomic."""
        return HostShmHeap._Locked(self._lock_fds[r], self._mutexes[r])

    def close(self) -> None:
        control.host_barrier()
        for fd in self._lock_fds.values():
            os.close(fd)
        self._lock_fds = {}
        self._maps = {}
        try:
            os.unlink(self._paths[self.rank])
        except FileNotFoundError:
            pass


class CudaHeap(SymmetricHeap):
    """GPU symmetric heap backed by the native extension."""

    def __init__(self, device: torch.device, nbytes: Optional[int] = None):
        from .. import _ext

        ext = _ext.load()
        self._ext = ext
        self.device = torch.device(device)
        self.rank, self.world = control.rank(), control.world_size()
        self.node = control.node_ranks()
        # the native heap spans one node: it knows ranks by their index within the node
        li, lw = self.rank - self.node[0], len(self.node)
        self.nbytes = _round_up(nbytes or config.symmetric_size("cuda"), 2 << 20)
        self.mode = config.heap_mode()
        token = f"{control.job_token()}_n{self.node[0]}"
        dev_index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        try:
            self._h = ext.heap_create(li, lw, dev_index, self.nbytes, self.mode, token)
        except RuntimeError as e:
            if self.mode != "vmm":
                raise
            logger.warning("virtual-memory heap unavailable (%s); falling back to CUDA-IPC slab", e)
            self.mode = "ipc"
            self.nbytes = min(self.nbytes, config.parse_size(os.environ.get("ODC_IPC_SLAB_SIZE", "8G")))
            self._h = ext.heap_create(li, lw, dev_index, self.nbytes, self.mode, token)
        # every rank must agree on the mode (a fallback on one rank only would desynchronise offsets)
        modes = control.all_gather_object(self.mode)
        if len(set(modes)) != 1:
            raise RuntimeError(f"ranks disagree on the heap mode: {modes}")
        if self.mode == "ipc":
            handles = control.all_gather_object(ext.heap_ipc_handle(self._h))
            for r, hb in enumerate(handles):
                if r != self.rank and self.is_local(r):
                    ext.heap_ipc_open(self._h, r - self.node[0], hb)
        control.host_barrier()  # all sockets bound / all slabs opened
        self._alloc = OffsetAllocator(self.nbytes)
        self._mapped = self.nbytes if self.mode == "ipc" else 0
        self._bases = {r: ext.heap_base(self._h, r - self.node[0]) for r in self.node}

    def alloc(self, nbytes: int) -> int:
        off = self._alloc.alloc(nbytes)
        need = self._alloc.high_water
        if need > self._mapped:
            # grow in steps so that many small allocations do not each pay an fd exchange
            step = max(need - self._mapped, 256 << 20)
            new_size = min(_round_up(self._mapped + step, 2 << 20), self.nbytes)
            self._ext.heap_grow(self._h, new_size)  # collective: exchanges fds with every peer
            self._mapped = new_size
        return off

    def free(self, offset: int) -> None:
        self._alloc.release(offset)  # physical pages stay mapped for reuse

    def local(self, offset, numel, dtype):
        return self.peer(self.rank, offset, numel, dtype)

    def peer(self, r, offset, numel, dtype):
        nb = numel * torch.empty((), dtype=dtype).element_size()
        if offset < 0 or offset + nb > self._mapped:
            raise IndexError(f"heap view [{offset}, {offset + nb}) outside mapped {self._mapped} bytes")
        self._check_local(r)
        return self._ext.tensor_from_ptr(self._bases[r] + offset, numel, dtype, self.device.index or 0)

    def peer_ptr(self, r, offset):
        self._check_local(r)
        return self._bases[r] + offset

    def offset_of(self, tensor):
        p = tensor.data_ptr()
        b = self._bases[self.rank]
        if b <= p < b + self.nbytes:
            return p - b
        return None

    @property
    def mapped_bytes(self) -> int:
        return self._mapped

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        control.host_barrier()
        self._ext.heap_destroy(self._h)
        self._h = None
        control.host_barrier()


def create_heap(device: torch.device, nbytes: Optional[int] = None) -> SymmetricHeap:
    device = torch.device(device)
    if device.type == "cuda":
        return CudaHeap(device, nbytes)
    return HostShmHeap(nbytes)
