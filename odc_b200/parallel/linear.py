"""A linear layer whose weight never exists unsharded outside the kernels that need it.

Rows of ``W [out, in]`` are split evenly over the group; each rank keeps its fp32 master rows, a
compute-precision copy in the symmetric heap (what peers pull) and an fp32 gradient accumulator in
the heap (what peers push into).  Forward is ONE kernel (``gather_linear``: shards stream in while
the GEMM runs), the weight-gradient is ONE kernel (``wgrad_scatter``: tiles are reduced into their
owners from the GEMM epilogue), and the input gradient is ONE kernel too (``gather_dgrad``: the
shards are pulled again while the k-loop follows their arrival) unless ``keep_weight=True`` keeps
the assembled weight from the forward pass.  No rank waits for another between ``start_minibatch``
and ``finish_minibatch``.

Gradient synchronisation can be deferred (``set_requires_gradient_sync(False)``, the same switch
FSDP2 modules have): weight gradients are then accumulated unsharded, in fp32, on the producing
rank, and pushed to their owners by the first later backward that runs with synchronisation on
(or by ``finish_minibatch``), so a minibatch of n microbatches crosses NVLink once instead of n times.

This is the on-demand design applied at layer level instead of through FSDP's hooks; it covers the
same two hot paths the reference patches into FSDP (odc/fsdp/fsdp2.py:218-313 and 607-742).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .. import ops
from ..ops import fused
from ..primitives import ReductionService
from ..runtime import control
from ..runtime.registry import SymmBufferRegistry

_layers: List["OdcLinear"] = []
_params: List["ShardedParameter"] = []
_reduction: Optional[ReductionService] = None
_next_id = 0
_sync_grads = True
_replicate_pg = None   # HSDP: the group of ranks that hold the same rows as this one (None: no replication)


def _service() -> ReductionService:
    global _reduction
    if _reduction is None:
        _reduction = ReductionService(accumulation_dtype=torch.float32)
    return _reduction


def set_replicate_group(pg) -> None:
    """Hybrid sharding: parameters are sharded over their own group and replicated over ``pg``.  Gradients are
    pushed to the owners inside the shard group during the minibatch and summed over ``pg`` once, after the
    per-minibatch synchronisation (the reference defers the replicate-dimension all-reduce the same way,
    odc/fsdp/fsdp2.py:849-882).  Set before the parameters are created."""
    global _replicate_pg
    _replicate_pg = pg


def replicas() -> int:
    return 1 if _replicate_pg is None else dist.get_world_size(_replicate_pg)


def set_requires_gradient_sync(flag: bool) -> None:
    """False: following backward passes accumulate weight gradients locally instead of pushing them to the owners."""
    global _sync_grads
    _sync_grads = bool(flag)


def requires_gradient_sync() -> bool:
    return _sync_grads


class ShardedParameter:
    """fp32 master rows + compute-precision heap copy + fp32 heap accumulator of one row-sharded matrix."""

    def __init__(self, name: str, full_shape, pg=None, device=None, init_std: float = 0.02, seed: int = 0,
                 full: Optional[torch.Tensor] = None, lowp_dtype: torch.dtype = torch.bfloat16):
        reg = SymmBufferRegistry.get_instance()
        self.name = name
        self.pg = pg
        self.ranks = control.group_ranks(pg)
        self.world = len(self.ranks)
        self.index = self.ranks.index(control.rank())
        self.out_features, self.in_features = int(full_shape[0]), int(full_shape[1])
        self.rows_per_rank = math.ceil(self.out_features / self.world)
        if self.out_features >= 128 * self.world:
            # whole 128-row output tiles per owner: the weight-gradient epilogue then reduces with bulk tensor
            # operations, one owner per tile (the padding rows stay zero)
            self.rows_per_rank = (self.rows_per_rank + 127) // 128 * 128
        device = torch.device(device) if device is not None else reg.heap.device
        lo, hi = self.index * self.rows_per_rank, (self.index + 1) * self.rows_per_rank
        self.master = torch.zeros(self.rows_per_rank, self.in_features, dtype=torch.float32, device=device)
        if full is None:
            gen = torch.Generator(device="cpu").manual_seed(seed)
            full = torch.randn(self.world * self.rows_per_rank, self.in_features, generator=gen) * init_std
            full[self.out_features:] = 0
        n = max(0, min(hi, full.shape[0], self.out_features) - lo)
        if n > 0:
            self.master[:n].copy_(full[lo:lo + n])
        self.lowp = reg.allocate_symm_buffer(f"odc_linear_w_{name}", (self.rows_per_rank, self.in_features), lowp_dtype)
        self.lowp.copy_(self.master)
        self.key = f"odc_linear_{name}"
        self.acc = _service().register(self.key, self.rows_per_rank * self.in_features, torch.float32, pg)
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        self.grad_scale = 1.0 / (self.world * replicas())
        # deferred synchronisation: unsharded fp32 gradient of this rank's own microbatches
        self.local_grad: Optional[torch.Tensor] = None
        self.local_dirty = False
        self.push_event = None
        _params.append(self)

    # -- views -----------------------------------------------------------------------------------------
    def grad(self) -> torch.Tensor:
        return self.acc.view(self.rows_per_rank, self.in_features)

    def flat(self):
        """``(master, accumulator, m, v, low-precision copy)`` as flat tensors, for the optimizer."""
        return self.master.view(-1), self.acc, self.m.view(-1), self.v.view(-1), self.lowp.view(-1)

    def local_buffer(self) -> torch.Tensor:
        if self.local_grad is None:
            self.local_grad = torch.zeros(self.world * self.rows_per_rank, self.in_features, dtype=torch.float32,
                                          device=self.master.device)
        return self.local_grad

    def wait_push(self) -> None:
        """Order the current stream after the last push of the local buffer (which zeroes it on a side stream)."""
        if self.push_event is not None:
            torch.cuda.current_stream().wait_event(self.push_event)
            self.push_event = None

    def push_local(self, side_stream: bool = False) -> None:
        """Add the locally accumulated gradient into the owners' accumulators (one-sided) and clear it."""
        if not self.local_dirty or self.local_grad is None:
            return
        buf = self.local_grad
        stream = control.get_comm_stream() if (side_stream and buf.is_cuda) else None
        if stream is not None:
            cur = torch.cuda.current_stream()
            stream.wait_stream(cur)
            with torch.cuda.stream(stream):
                _service().scatter_accumulate(self.key, buf.view(-1), self.pg, scale=self.grad_scale)
                buf.zero_()
                self.push_event = stream.record_event()
        else:
            _service().scatter_accumulate(self.key, buf.view(-1), self.pg, scale=self.grad_scale)
            buf.zero_()
        self.local_dirty = False

    # -- whole-matrix access (collective; checkpoints and tests) ------------------------------------------
    def full_master(self) -> torch.Tensor:
        parts = [torch.empty_like(self.master) for _ in range(self.world)]
        if self.world > 1:
            dist.all_gather(parts, self.master.contiguous(), group=self.pg)
        else:
            parts[0] = self.master
        return torch.cat(parts)[:self.out_features].clone()

    def _full_of(self, t: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(t) for _ in range(self.world)]
        if self.world > 1:
            dist.all_gather(parts, t.contiguous(), group=self.pg)
        else:
            parts[0] = t
        return torch.cat(parts)[:self.out_features].clone()

    def load_full(self, full: torch.Tensor, m: Optional[torch.Tensor] = None, v: Optional[torch.Tensor] = None) -> None:
        lo = self.index * self.rows_per_rank
        for dst, src in ((self.master, full), (self.m, m), (self.v, v)):
            if src is None:
                continue
            dst.zero_()
            n = max(0, min(lo + self.rows_per_rank, self.out_features) - lo)
            if n > 0:
                dst[:n].copy_(src[lo:lo + n])
        self.lowp.copy_(self.master)


class _OdcLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, residual, layer):
        p = layer.weight
        if p.world == 1:
            w_full = p.lowp[:p.out_features]      # the shard is the matrix: nothing to pull
            x2 = x.reshape(-1, x.shape[-1])
            res2 = None if residual is None else residual.reshape(-1, p.out_features)
            if x2.is_cuda:
                y = ops.gemm(x2, w_full, "nt", bias=bias, residual=res2)
            else:
                y = torch.nn.functional.linear(x2, w_full.to(x2.dtype), bias)
                y = y if res2 is None else y + res2
            y = y.view(*x.shape[:-1], p.out_features)
        else:
            y, w_full = fused.gather_linear(x, p.lowp, p.out_features, p.pg, bias, residual)
        ctx.layer = layer
        ctx.has_bias = bias is not None
        if layer.keep_weight and p.world > 1:
            ctx.save_for_backward(x, w_full)
        else:
            ctx.save_for_backward(x)  # the assembled weight is dropped; backward pulls the shards again
        return y

    @staticmethod
    def backward(ctx, dy):
        layer = ctx.layer
        p = layer.weight
        saved = ctx.saved_tensors  # read once: activation checkpointing recomputes on the first access only
        x = saved[0]
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = None
        if ctx.needs_input_grad[0]:
            if p.world == 1 or layer.keep_weight:
                w_full = p.lowp[:p.out_features] if p.world == 1 else saved[1]
                dx = ops.gemm(dy2, w_full, "nn") if dy2.is_cuda else dy2 @ w_full.to(dy2.dtype)
                dx = dx.view(x.shape)
            else:
                dx = fused.gather_dgrad(dy2, p.lowp, p.out_features, p.pg)[0].view(x.shape)
        accumulate_weight_grad(p, dy2, x2)
        db = None
        if ctx.has_bias and ctx.needs_input_grad[1]:
            db = dy2.float().sum(0).to(dy.dtype)
        dres = dy if ctx.needs_input_grad[2] else None
        return dx, db, dres, None


def accumulate_weight_grad(p: ShardedParameter, dy2: torch.Tensor, x2: torch.Tensor) -> None:
    """``dW = dy2.T @ x2`` of one microbatch: straight into the owners (fused epilogue), or into the local buffer."""
    if _sync_grads:
        fused.wgrad_scatter(dy2, x2, _service(), p.key, 0, p.rows_per_rank, p.pg, p.grad_scale)
        p.push_local()  # what earlier microbatches accumulated locally follows
        return
    p.wait_push()
    buf = p.local_buffer()
    if dy2.is_cuda:
        ops.gemm(dy2, x2.contiguous(), "tn", out=buf[:p.out_features], accumulate=True)
    else:
        buf[:p.out_features] += dy2.float().t() @ x2.float()
    p.local_dirty = True


class OdcLinear(nn.Module):
    def __init__(self, in_features: int, out_features: int, pg=None, name: Optional[str] = None, seed: int = 0,
                 init_std: float = 0.02, keep_weight: bool = False, full: Optional[torch.Tensor] = None,
                 lowp_dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        global _next_id
        name = name or f"l{_next_id}"
        _next_id += 1
        self.weight = ShardedParameter(name, (out_features, in_features), pg, init_std=init_std, seed=seed, full=full,
                                       lowp_dtype=lowp_dtype)
        self.bias = None
        # False: only the shard outlives the forward kernel (memory of a sharded model); the input
        # gradient is then the gather-fused GEMM.  True trades out*in*2 bytes per layer for one transfer.
        self.keep_weight = keep_weight
        _layers.append(self)

    @property
    def grad_scale(self) -> float:
        return self.weight.grad_scale

    def forward(self, x, bias=None, residual=None):
        return _OdcLinearFn.apply(x, bias if bias is not None else self.bias, residual, self)


def sharded_parameters() -> List[ShardedParameter]:
    return list(_params)


def start_minibatch() -> None:
    """Zero the accumulators and publish the freshly written low-precision rows (collective)."""
    _service().clear_accumulations()
    if torch.cuda.is_available():
        torch.cuda.current_stream().synchronize()
    control.host_barrier()


def flush_local_grads() -> None:
    """Push whatever is still accumulated locally (a minibatch whose last backward ran with synchronisation off)."""
    for p in _params:
        p.push_local()
        p.wait_push()


@torch.no_grad()
def finish_minibatch(lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                     step: int = 1, optimizer_step: bool = True) -> None:
    """Wait for all contributions (collective), then AdamW on every layer's own rows."""
    flush_local_grads()
    _service().sync()
    if _replicate_pg is not None and replicas() > 1:
        for acc in _service().accumulations.values():   # one all-reduce per matrix and minibatch
            dist.all_reduce(acc, group=_replicate_pg)
    if not optimizer_step:
        return
    for layer in _layers:
        master, acc, m, v, lowp = layer.weight.flat()
        ops.fused_adamw_(master, acc, m, v, lowp, lr, betas[0], betas[1], eps, weight_decay, step, 1.0)


def reset() -> None:
    global _reduction, _next_id, _sync_grads, _replicate_pg
    _layers.clear()
    _params.clear()
    _reduction = None
    _next_id = 0
    _sync_grads = True
    _replicate_pg = None
