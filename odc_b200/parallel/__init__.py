"""Native sharded layers that use the fused compute+communication kernels directly."""
from .linear import OdcLinear, ShardedParameter, finish_minibatch, reset, start_minibatch

__all__ = ["OdcLinear", "ShardedParameter", "start_minibatch", "finish_minibatch", "reset"]
