"""GEMMs fused with the on-demand primitives (single launches).

``gather_linear``: ``y = x @ W.T`` where ``W`` is row-sharded over a group and lives in the
symmetric heap; the kernel pulls the owners' shards into a local buffer panel by panel while the
tensor cores already multiply the panels that have landed.  Returns the assembled weight too, so
the backward pass (or a later microbatch) can reuse it without another transfer.

``gather_dgrad``: ``dx = dy @ W`` with the same sharded ``W``; the shards are pulled again instead of
keeping the assembled weight alive between forward and backward.

``wgrad_scatter``: ``dW = dy.T @ x`` whose epilogue adds every output tile into the owning rank's
fp32 accumulator and signals arrival, with the same bookkeeping as
``ReductionService.scatter_accumulate`` (one dispatched contribution per owner per call).

On CPU both fall back to the plain statement of the op over the host-shm heap so that the
multi-rank logic is testable without a GPU.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..primitives import ReductionService
from ..runtime import control
from ..runtime.registry import SymmBufferRegistry


_transports = {}


def _spans_nodes(reg: SymmBufferRegistry, ranks) -> bool:
    return any(not reg.heap.is_local(r) for r in ranks)


def _gather_weight(reg: SymmBufferRegistry, weight_shard: torch.Tensor, ranks, out_features: int) -> torch.Tensor:
    """Unfused assembly of ``W`` for groups that reach other nodes (their shards are not mapped here)."""
    from ..runtime.transport import make_transport
    tr = _transports.get(id(reg))
    if tr is None or tr.registry is not reg:
        tr = _transports[id(reg)] = make_transport(reg)
    rows_per, K = weight_shard.shape
    w = torch.empty(len(ranks) * rows_per, K, dtype=weight_shard.dtype, device=weight_shard.device)
    me = control.rank()
    tr.gather(w.view(len(ranks), -1), weight_shard, ranks, ranks.index(me) if me in ranks else 0)
    return w[:out_features]


def gather_linear(x: torch.Tensor, weight_shard: torch.Tensor, out_features: int,
                  pg: Optional[dist.ProcessGroup] = None, bias: Optional[torch.Tensor] = None,
                  residual: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``weight_shard``: this rank's ``[rows_per_rank, K]`` rows of ``W`` (a symmetric-heap tensor).

    ``bias`` and ``residual`` (``[..., out_features]``) are added in the kernel's epilogue."""
    reg = SymmBufferRegistry.get_instance()
    ranks = control.group_ranks(pg)
    me = control.rank()
    rows_per, K = weight_shard.shape
    x2 = x.reshape(-1, x.shape[-1])
    res2 = None if residual is None else residual.reshape(-1, out_features)
    if _spans_nodes(reg, ranks):
        from . import gemm
        w_full = _gather_weight(reg, weight_shard, ranks, out_features)
        if x2.is_cuda:
            y = gemm(x2, w_full, "nt", bias=bias, residual=res2)
        else:
            y = torch.nn.functional.linear(x2, w_full.to(x2.dtype), bias)
            y = y if res2 is None else y + res2
    elif x2.is_cuda:
        from .. import _ext
        from . import _count
        table = reg.peer_ptr_table(weight_shard, ranks)
        w_full = torch.empty(out_features, K, dtype=weight_shard.dtype, device=x.device)
        y = _ext.load().gemm_gather(x2, table, w_full, bias, rows_per, ranks.index(me) if me in ranks else 0, res2)
        _count()
    else:
        peers = reg.get_peer_tensors(weight_shard)
        w_full = torch.cat([peers[r] for r in ranks], dim=0)[:out_features].clone()
        y = torch.nn.functional.linear(x2, w_full.to(x2.dtype), bias)
        y = y if res2 is None else y + res2
    return y.view(*x.shape[:-1], out_features), w_full


def gather_dgrad(dy: torch.Tensor, weight_shard: torch.Tensor, out_features: int,
                 pg: Optional[dist.ProcessGroup] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``dx = dy @ W`` with ``W [out_features, K]`` row-sharded as in :func:`gather_linear`.

    The gathered rows are the reduction dimension here: the k-loop of each CTA's first tile walks the
    256-row groups as they land, later tiles read the assembled weight.  Returns ``(dx, w_full)``.
    """
    reg = SymmBufferRegistry.get_instance()
    ranks = control.group_ranks(pg)
    rows_per, K = weight_shard.shape
    dy2 = dy.reshape(-1, dy.shape[-1])
    if _spans_nodes(reg, ranks):
        from . import gemm
        w_full = _gather_weight(reg, weight_shard, ranks, out_features)
        dx = gemm(dy2.contiguous(), w_full, "nn") if dy2.is_cuda else dy2 @ w_full.to(dy2.dtype)
    elif dy2.is_cuda:
        from .. import _ext
        from . import _count
        table = reg.peer_ptr_table(weight_shard, ranks)
        w_full = torch.empty(out_features, K, dtype=weight_shard.dtype, device=dy.device)
        if dy2.stride(1) != 1:
            dy2 = dy2.contiguous()
        me = control.rank()
        dx = _ext.load().gemm_gather_dgrad(dy2, table, w_full, rows_per, ranks.index(me) if me in ranks else 0)
        _count()
    else:
        peers = reg.get_peer_tensors(weight_shard)
        w_full = torch.cat([peers[r] for r in ranks], dim=0)[:out_features].clone()
        dx = dy2 @ w_full.to(dy2.dtype)
    return dx.view(*dy.shape[:-1], K), w_full


def wgrad_scatter(dy: torch.Tensor, x: torch.Tensor, reduction: ReductionService, key, param_offset: int,
                  rows_per_rank: int, pg: Optional[dist.ProcessGroup] = None, scale: float = 1.0) -> None:
    """Add ``scale * dy.T @ x`` (shape ``[n_out, k_in]``, rows split ``rows_per_rank`` per owner) into ``key``."""
    ranks = control.group_ranks(pg)
    acc = reduction.scatter_target(key)
    dy2 = dy.reshape(-1, dy.shape[-1])
    x2 = x.reshape(-1, x.shape[-1])
    n_out, k_in = dy2.shape[1], x2.shape[1]
    if param_offset + rows_per_rank * k_in > acc.numel():
        raise ValueError("parameter does not fit in the accumulator at this offset")
    if _spans_nodes(reduction.registry, ranks):
        # unfused: form the gradient locally, then hand the rows to the transport (same-node owners over the
        # mapped heap, the rest through the inter-node path)
        if dy2.is_cuda:
            from . import gemm
            dw = gemm(dy2.contiguous(), x2.contiguous(), "tn", out_dtype=torch.float32)
        else:
            dw = dy2.float().t() @ x2.float()
        pad = rows_per_rank * len(ranks) - n_out
        if pad:
            dw = torch.cat([dw, dw.new_zeros(pad, k_in)])
        me = control.rank()
        target = acc[param_offset:param_offset + rows_per_rank * k_in]
        reduction.transport.scatter_add(dw.view(len(ranks), -1), target, reduction.counter, ranks,
                                        ranks.index(me) if me in ranks else 0, scale)
        reduction.note_dispatch(ranks)
    elif dy2.is_cuda:
        from .. import _ext
        from . import _count
        reg = reduction.registry
        if acc.dtype != torch.float32:
            raise ValueError("the fused weight-gradient path accumulates in fp32")
        ext = _ext.load()
        dy2, x2 = dy2.contiguous(), x2.contiguous()
        done = False
        if os.environ.get("ODC_WGRAD_SCATTER", "tma") == "tma":
            # output boxes staged in shared memory and added into the owners by the TMA unit; needs
            # rows_per_rank % 128 == 0 and at most 8 owners, otherwise the per-thread red.add variant runs
            me = control.rank()
            done = ext.gemm_wgrad_scatter_tma(dy2, x2, reg.peer_ptrs(acc, ranks), reg.peer_ptr_table(reduction.counter, ranks),
                                              param_offset, rows_per_rank, scale, ranks.index(me) if me in ranks else 0)
        if not done:
            ext.gemm_wgrad_scatter(dy2, x2, reg.peer_ptr_table(acc, ranks), reg.peer_ptr_table(reduction.counter, ranks),
                                   param_offset, rows_per_rank, scale)
        _count()
        reduction.note_dispatch(ranks)
    else:
        dw = (dy2.float().t() @ x2.float()) * scale
        pad = rows_per_rank * len(ranks) - n_out
        if pad:
            dw = torch.cat([dw, dw.new_zeros(pad, k_in)])
        accs = reduction.registry.get_peer_tensors(acc)
        ctrs = reduction.registry.get_peer_tensors(reduction.counter)
        heap = reduction.registry.heap
        for i, r in enumerate(ranks):
            with heap.owner_lock(r):
                accs[r][param_offset:param_offset + rows_per_rank * k_in] += \
                    dw[i * rows_per_rank:(i + 1) * rows_per_rank].reshape(-1).to(acc.dtype)
                ctrs[r][0] += 1
        reduction.note_dispatch(ranks)
