"""Native sharded layers that use the fused compute+communication kernels directly."""
from .decoder import FusedDecoderLM, FusedOptimizer
from .linear import (OdcLinear, ShardedParameter, finish_minibatch, requires_gradient_sync, reset,
                     set_requires_gradient_sync, sharded_parameters, start_minibatch)

__all__ = ["OdcLinear", "ShardedParameter", "FusedDecoderLM", "FusedOptimizer", "start_minibatch", "finish_minibatch",
           "reset", "set_requires_gradient_sync", "requires_gradient_sync", "sharded_parameters"]
