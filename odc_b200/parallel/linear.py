"""A linear layer whose weight never exists unsharded outside the kernels that need it.

Rows of ``W [out, in]`` are split evenly over the group; each rank keeps its fp32 master rows, a
bf16 copy in the symmetric heap (what peers pull) and an fp32 gradient accumulator in the heap
(what peers push into).  Forward is ONE kernel (``gather_linear``: shards stream in while the
GEMM runs), the weight-gradient is ONE kernel (``wgrad_scatter``: tiles are reduced into their
owners from the GEMM epilogue), and the input gradient is ONE kernel too (``gather_dgrad``: the
shards are pulled again while the k-loop follows their arrival) unless ``keep_weight=True`` keeps
the assembled weight from the forward pass.  No rank waits for another between ``start_minibatch`` and ``finish_minibatch``.

This is the on-demand design applied at layer level instead of through FSDP's hooks; it covers the
same two hot paths the reference patches into FSDP (odc/fsdp/fsdp2.py:218-313 and 607-742).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn as nn

from .. import ops
from ..ops import fused
from ..primitives import ReductionService
from ..runtime import control
from ..runtime.registry import SymmBufferRegistry

_layers: List["OdcLinear"] = []
_reduction: Optional[ReductionService] = None
_next_id = 0


def _service() -> ReductionService:
    global _reduction
    if _reduction is None:
        _reduction = ReductionService(accumulation_dtype=torch.float32)
    return _reduction


class ShardedParameter:
    """fp32 master rows + bf16 heap copy + fp32 heap accumulator of one row-sharded matrix."""

    def __init__(self, name: str, full_shape, pg=None, device=None, init_std: float = 0.02, seed: int = 0):
        reg = SymmBufferRegistry.get_instance()
        self.pg = pg
        self.ranks = control.group_ranks(pg)
        self.world = len(self.ranks)
        self.index = self.ranks.index(control.rank())
        self.out_features, self.in_features = full_shape
        self.rows_per_rank = math.ceil(self.out_features / self.world)
        device = device or reg.heap.device
        gen = torch.Generator(device="cpu").manual_seed(seed)
        full = torch.randn(self.world * self.rows_per_rank, self.in_features, generator=gen) * init_std
        full[self.out_features:] = 0
        mine = full[self.index * self.rows_per_rank:(self.index + 1) * self.rows_per_rank]
        self.master = mine.to(device=device, dtype=torch.float32).contiguous()
        self.lowp = reg.allocate_symm_buffer(f"odc_linear_w_{name}", (self.rows_per_rank, self.in_features),
                                             torch.bfloat16)
        self.lowp.copy_(self.master)
        self.key = f"odc_linear_{name}"
        self.acc = _service().register(self.key, self.rows_per_rank * self.in_features, torch.float32, pg)
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)

    def grad(self) -> torch.Tensor:
        return self.acc.view(self.rows_per_rank, self.in_features)


class _OdcLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, layer):
        p = layer.weight
        y, w_full = fused.gather_linear(x, p.lowp, p.out_features, p.pg, layer.bias)
        ctx.layer = layer
        if layer.keep_weight:
            ctx.save_for_backward(x, w_full)
        else:
            ctx.save_for_backward(x)  # the assembled weight is dropped; backward pulls the shards again
        return y

    @staticmethod
    def backward(ctx, dy):
        layer = ctx.layer
        p = layer.weight
        x = ctx.saved_tensors[0]
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = None
        if ctx.needs_input_grad[0]:
            if not layer.keep_weight:
                dx = fused.gather_dgrad(dy2, p.lowp, p.out_features, p.pg)[0].view(x.shape)
            else:
                w_full = ctx.saved_tensors[1]
                dx = ops.gemm(dy2, w_full, "nn").view(x.shape) if dy2.is_cuda else (dy2 @ w_full.to(dy2.dtype)).view(x.shape)
        fused.wgrad_scatter(dy2, x2, _service(), p.key, 0, p.rows_per_rank, p.pg, layer.grad_scale)
        return dx, None


class OdcLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, pg=None, name: Optional[str] = None, seed: int = 0,
                 init_std: float = 0.02, keep_weight: bool = False):
        super().__init__()
        global _next_id
        name = name or f"l{_next_id}"
        _next_id += 1
        self.weight = ShardedParameter(name, (out_features, in_features), pg, init_std=init_std, seed=seed)
        self.bias = None
        # False: only the shard outlives the forward kernel (memory of a sharded model); the input
        # gradient is then the gather-fused GEMM.  True trades out*in*2 bytes per layer for one transfer.
        self.keep_weight = keep_weight
        self.grad_scale = 1.0 / self.weight.world
        _layers.append(self)

    def forward(self, x):
        return _OdcLinearFn.apply(x, self)


def start_minibatch() -> None:
    """Zero the accumulators and publish the freshly written bf16 rows (collective)."""
    _service().clear_accumulations()
    if torch.cuda.is_available():
        torch.cuda.current_stream().synchronize()
    control.host_barrier()


@torch.no_grad()
def finish_minibatch(lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                     step: int = 1) -> None:
    """Wait for all contributions (collective), then AdamW on every layer's own rows."""
    _service().sync()
    for layer in _layers:
        p = layer.weight
        ops.fused_adamw_(p.master.view(-1), p.acc, p.m.view(-1), p.v.view(-1), p.lowp.view(-1), lr, betas[0], betas[1],
                         eps, weight_decay, step, 1.0)


def reset() -> None:
    global _reduction, _next_id
    _layers.clear()
    _reduction = None
    _next_id = 0
