from . import fsdp1, fsdp2

__all__ = ["fsdp1", "fsdp2"]
