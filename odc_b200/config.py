"""Environment-variable configuration.

The reference is configured purely through environment variables and function
arguments (odc/primitives/utils.py:212-219, launch.sh:130-141); this module keeps
that style and gathers every knob in one place.  Values are read when asked for,
not at import, so tests can change them with ``monkeypatch.setenv``.
"""
from __future__ import annotations

import os

_SUFFIX = {"k": 1 << 10, "m": 1 << 20, "g": 1 << 30, "t": 1 << 40}


def parse_size(text: str) -> int:
    """Parse ``"5G"``, ``"512M"``, ``"1073741824"`` … into bytes."""
    t = text.strip().lower()
    if t.endswith("ib"):
        t = t[:-2]
    elif t.endswith("b") and len(t) > 1 and not t[-2].isdigit():
        t = t[:-1]
    mult = 1
    if t and t[-1] in _SUFFIX:
        mult = _SUFFIX[t[-1]]
        t = t[:-1]
    return int(float(t) * mult)


def max_buffer_elems() -> int:
    """Staging cap in ELEMENTS (``ODC_MAX_BUFFER_SIZE``; <=0 disables splitting).

    Same variable, unit and default as the reference (odc/primitives/utils.py:216-219).
    """
    return int(os.environ.get("ODC_MAX_BUFFER_SIZE", str(64 * (1 << 20))))


def symmetric_size(device_type: str) -> int:
    """Bytes of symmetric address space reserved per rank.

    ``ODC_SYMMETRIC_SIZE`` wins; ``NVSHMEM_SYMMETRIC_SIZE`` is honoured so launch
    scripts written for the reference (launch.sh:135) keep working.  On CUDA this
    is only a virtual-address reservation (physical pages are mapped as buffers
    are allocated), so the default is generous.
    """
    for name in ("ODC_SYMMETRIC_SIZE", "NVSHMEM_SYMMETRIC_SIZE"):
        if name in os.environ:
            return parse_size(os.environ[name])
    return (64 << 30) if device_type == "cuda" else (1 << 30)


def heap_mode() -> str:
    """``vmm`` (cuMem virtual memory + POSIX fd export) or ``ipc`` (cudaMalloc slab + cudaIpc)."""
    return os.environ.get("ODC_HEAP_MODE", "vmm").lower()


def wait_timeout_ms() -> int:
    """Budget of every bounded wait (device spin or host poll) before it reports an error."""
    return int(os.environ.get("ODC_WAIT_TIMEOUT_MS", "60000"))


def sync_by_posting() -> bool:
    """``ODC_SYNC_POSTING=0``: ``ReductionService.sync`` always exchanges dispatch counts on the host.

    By default a ``sync`` that carries no payload makes the counts known by one-sided stores into the owners.
    """
    return os.environ.get("ODC_SYNC_POSTING", "1") not in ("0", "false")


def heartbeat_s() -> float:
    """``ODC_HEARTBEAT_S`` > 0: publish a host heartbeat every second and, before each once-per-minibatch
    synchronisation, treat a peer whose last beat is older than this many seconds as failed (0: off)."""
    return float(os.environ.get("ODC_HEARTBEAT_S", "0"))


def debug_bounds() -> bool:
    """Turn on offset/peer-index checks inside the communication kernels."""
    return os.environ.get("ODC_DEBUG_BOUNDS", "0") not in ("0", "", "false")


def deterministic() -> bool:
    """``ODC_DETERMINISTIC=1``: per-source slots on the owner, summed in rank order at ``sync`` (debugging aid).

    The default path adds every producer's rows into one accumulator with remote floating-point reductions,
    whose order across producers varies from run to run.
    """
    return os.environ.get("ODC_DETERMINISTIC", "0") not in ("0", "", "false")


def reduce_from_segments() -> bool:
    """``ODC_REDUCE_SEGMENTS=0``: FSDP2 flattens the gradients rank-major before the reduction (for A/B runs).

    By default the reduction reads the per-parameter gradient tensors directly.
    """
    return os.environ.get("ODC_REDUCE_SEGMENTS", "1") not in ("0", "false")


def local_world_size(default: int) -> int:
    """GPUs per node: ``RAY_LOCAL_WORLD_SIZE`` overrides ``LOCAL_WORLD_SIZE`` (utils.py:195-199)."""
    for name in ("RAY_LOCAL_WORLD_SIZE", "LOCAL_WORLD_SIZE"):
        if name in os.environ:
            return int(os.environ[name])
    return default


def nvtx_enabled() -> bool:
    return os.environ.get("ODC_NVTX", "1") not in ("0", "", "false")
