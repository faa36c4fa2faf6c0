from .gather import GatherService
from .scatter_accumulate import ReductionService
from .splitter import BufferSplitter

__all__ = ["GatherService", "ReductionService", "BufferSplitter"]
