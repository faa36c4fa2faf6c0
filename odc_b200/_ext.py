"""Loader of the in-tree native extension (``odc_b200/_C*.so``).

The extension is built by ``python -m odc_b200.build`` (or ``__graft_entry__.build()``) with
``-gencode arch=compute_100a,code=sm_100a``.  GPU code paths call :func:`load`, which raises if
the library is missing: there is no silent PyTorch fallback on a GPU.
"""
from __future__ import annotations

import glob
import importlib.util
import os

_mod = None


def so_path() -> str | None:
    here = os.path.dirname(os.path.abspath(__file__))
    hits = sorted(glob.glob(os.path.join(here, "_C*.so")))
    return hits[0] if hits else None


def available() -> bool:
    return so_path() is not None


def load():
    global _mod
    if _mod is None:
        path = so_path()
        if path is None:
            raise ImportError(
                "odc_b200 native extension not built: run `python -m odc_b200.build` "
                "(needs nvcc; cross-compiles for sm_100a without a GPU)")
        import torch  # noqa: F401  (libtorch symbols must be loaded first)

        spec = importlib.util.spec_from_file_location("odc_b200._C", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _mod = mod
    return _mod
