from .gather import GatherService
from .scatter_accumulate import ReductionService
from .splitter import BufferSplitter

__all__ = ["GatherService", "ReductionService", "BufferSplitter"]


def get_ipc_handle(tensor):
    """Serialised CUDA-IPC handle (+ offset inside its allocation) of a device tensor, for another process on the node.

    Counterpart of the reference's ``tensor_ipc.get_ipc_handle`` (csrc/tensor_ipc/tensor_ipc.cu:24-44); errors raise.
    The tensor must come from ``cudaMalloc``-style memory (not from the virtual-memory heap, whose buffers are shared
    through the heap itself).
    """
    from .. import _ext
    return _ext.load().get_ipc_handle(tensor)


def reconstruct_tensor(handle: bytes, shape, dtype):
    """Map a tensor exported by :func:`get_ipc_handle` in another process (csrc/tensor_ipc/tensor_ipc.cu:46-57)."""
    from .. import _ext
    return _ext.load().reconstruct_tensor(handle, list(shape), dtype)


__all__ += ["get_ipc_handle", "reconstruct_tensor"]
