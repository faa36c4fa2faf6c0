"""NVTX ranges that cost nothing on CPU (reference: odc/fsdp/fsdp2.py:54-61)."""
from __future__ import annotations

import contextlib

import torch
from torch.profiler import record_function

from .. import config


@contextlib.contextmanager
def nvtx_range(name: str):
    on = config.nvtx_enabled() and torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class nvtx_record_function(record_function):
    """``record_function`` that also opens an NVTX range, so FSDP phases show up in Nsight."""

    def __enter__(self):
        self._nvtx = config.nvtx_enabled() and torch.cuda.is_available()
        if self._nvtx:
            torch.cuda.nvtx.range_push(self.name)
        return super().__enter__()

    def __exit__(self, exc_type, exc_value, traceback):
        super().__exit__(exc_type, exc_value, traceback)
        if self._nvtx:
            torch.cuda.nvtx.range_pop()
