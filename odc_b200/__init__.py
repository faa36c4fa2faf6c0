"""odc_b200 — on-demand-communication FSDP for Blackwell (B200, sm_100a).

Public surface mirrors the reference package (odc/__init__.py:3-18): ``init_nvshmem``,
``finalize_distributed``, ``SymmBufferRegistry``, ``GatherService``, ``ReductionService`` and the
``fsdp`` sub-package (``fsdp1`` / ``fsdp2``).  ``init_nvshmem`` keeps its name for drop-in use
although the symmetric heap underneath is this package's own (CUDA virtual-memory handles
mapped into every rank), not NVSHMEM.
"""
from __future__ import annotations

import logging
from typing import Optional

import torch

from .primitives import BufferSplitter, GatherService, ReductionService
from .runtime import (SymmBufferRegistry, get_comm_stream, get_local_world_pg, get_local_world_size)
from .runtime import control as _control

logging.getLogger("odc_b200").addHandler(logging.NullHandler())

__version__ = "0.1.0"


def init_nvshmem(device: Optional[torch.device] = None, symmetric_size: Optional[int] = None) -> SymmBufferRegistry:
    """Create this rank's symmetric heap and map every peer's heap (collective).

    Call after ``torch.distributed.init_process_group`` (and ``torch.cuda.set_device`` on GPU),
    exactly where the reference calls ``odc.init_nvshmem()`` (odc/primitives/utils.py:18-49).
    With no process group the heap has a single rank, which is enough for single-GPU runs.
    """
    return SymmBufferRegistry.initialize(device, symmetric_size)


init_symmetric_heap = init_nvshmem


def finalize_distributed() -> None:
    """Free every symmetric buffer and unmap the heap (odc/primitives/utils.py:84-85)."""
    if SymmBufferRegistry.is_initialized():
        SymmBufferRegistry.get_instance().finalize()
    _control.reset_control_group()


__all__ = [
    "init_nvshmem", "init_symmetric_heap", "finalize_distributed", "SymmBufferRegistry", "GatherService",
    "ReductionService", "BufferSplitter", "get_comm_stream", "get_local_world_size", "get_local_world_pg",
]
