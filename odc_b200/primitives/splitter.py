"""Staging-size policy (``ODC_MAX_BUFFER_SIZE``).

Same arithmetic as the reference's ``BufferSplitter`` (odc/primitives/utils.py:212-242): the
cap is in ELEMENTS, a non-positive cap turns splitting off, the per-peer mailbox size is
rounded up to 64 elements.  Inside one NVLink domain the kernels write straight to their final
destination, so the cap only bounds how much one launch moves (and sizes inter-node staging).
"""
from __future__ import annotations

import math
from typing import Iterator, Sequence, Tuple

from .. import config


class BufferSplitter:
    def __init__(self, max_buffer_size: int | None = None):
        self.max_buffer_size = config.max_buffer_elems() if max_buffer_size is None else int(max_buffer_size)

    @property
    def enabled(self) -> bool:
        return self.max_buffer_size > 0

    def get_global_buffer_size(self, shape: Sequence[int]) -> int:
        numel = int(math.prod(shape))
        return numel if not self.enabled else min(self.max_buffer_size, numel)

    def get_local_buffer_size(self, shape: Sequence[int], world_size: int) -> int:
        numel = int(math.prod(shape))
        if not self.enabled:
            size = numel
        else:
            if self.max_buffer_size % world_size != 0:
                raise ValueError(
                    f"ODC_MAX_BUFFER_SIZE={self.max_buffer_size} must be a multiple of the group size {world_size}")
            size = min(self.max_buffer_size // world_size, numel)
        return (size + 63) // 64 * 64

    def segments(self, shard_numel: int, world_size: int) -> Iterator[Tuple[int, int]]:
        """``(start, length)`` pieces of a shard, each at most the per-peer buffer size."""
        if shard_numel == 0:
            return
        step = self.get_local_buffer_size((shard_numel,), world_size)
        step = max(step, 1)
        for start in range(0, shard_numel, step):
            yield start, min(step, shard_numel - start)
