"""On-demand communication for PyTorch FSDP1 (``FullyShardedDataParallel`` with flat parameters).

Public API of the reference (odc/fsdp/fsdp1.py:302-348): ``patch_fsdp1(reduce_dtype=None)`` before
any ``FSDP(...)`` is constructed, ``pre_minibatch_start(fsdp_model)`` once after construction and
after every optimizer step, ``pre_optimizer_step(fsdp_model)`` before ``optimizer.step()``,
``stop()``.  Supported: FULL_SHARD / SHARD_GRAD_OP with ``use_orig_params=False``, with or without
mixed precision; unsupported (asserted): communication hooks, HYBRID_SHARD, CPU offload.

How it works here:

* ``FlatParamHandle.shard`` places the rank's flat shard in the symmetric heap, so the optimizer
  updates memory that peers can read.
* With parameter mixed precision a second heap buffer holds the shard in the compute dtype,
  refreshed once per minibatch; ``_all_gather_flat_param`` becomes one ``gather`` launch that pulls
  compute-precision bytes (the reference pulls the original dtype and casts after the transfer,
  odc/fsdp/fsdp1.py:189-223).  The per-unshard low-precision copy of stock FSDP is skipped.
* ``_reduce_grad`` ``scatter_accumulate``-s the unsharded gradient where it lies (a flat gradient
  that does not divide by the group size is reduced as ragged pieces instead of being padded with
  a copy), folding the pre/post divide factors into the kernel's scale; nothing is attached to
  ``flat_param.grad`` until ``pre_optimizer_step`` has waited for all contributions, and then it
  is the accumulator itself (or its cast to the shard's dtype), not a copy.
"""
from __future__ import annotations

import logging
from typing import Any, Dict, List, Optional

import torch
import torch.distributed.fsdp._runtime_utils as _ru
import torch.nn.functional as F
import torch.distributed.fsdp._traversal_utils as _tu
from torch.distributed.fsdp._common_utils import _FSDPState
from torch.distributed.fsdp._flat_param import FlatParamHandle, HandleShardingStrategy

from .. import config
from ..primitives import GatherService, ReductionService
from ..runtime import control
from ..runtime.registry import SymmBufferRegistry
from ..utils.nvtx import nvtx_range

logger = logging.getLogger("odc_b200")


class _State:
    patched = False
    reduce_dtype: Optional[torch.dtype] = None
    originals: Dict[str, Any] = {}
    reduction: Optional[ReductionService] = None
    gather: Optional[GatherService] = None
    next_index = 0
    in_shard: Optional[FlatParamHandle] = None
    touched: set = set()   # keys of flat parameters this rank reduced a gradient for in this minibatch
    used: set = set()      # keys some rank reduced a gradient for, as of the last pre_optimizer_step


_S = _State


def get_reduction_service():
    return _S.reduction


def get_gather_service():
    return _S.gather


def _services():
    if _S.reduction is None:
        _S.reduction = ReductionService(accumulation_dtype=_S.reduce_dtype)
        _S.gather = GatherService()
    return _S.reduction, _S.gather


def _check_supported(handle: FlatParamHandle) -> None:
    if handle._sharding_strategy in (HandleShardingStrategy.HYBRID_SHARD, HandleShardingStrategy._HYBRID_SHARD_ZERO2):
        raise AssertionError("on-demand FSDP1 does not support HYBRID_SHARD (use FSDP2 for HSDP)")
    if handle._offload_params:
        raise AssertionError("on-demand FSDP1 does not support CPU offload")
    if handle._use_orig_params:
        raise AssertionError("on-demand FSDP1 requires use_orig_params=False")


# ------------------------------------------------------------------------------------------
# shard -> symmetric heap
# ------------------------------------------------------------------------------------------
def _shard(self: FlatParamHandle):
    if not self.uses_sharded_strategy:
        return _S.originals["shard"](self)
    _check_supported(self)
    _S.in_shard = self
    try:
        return _S.originals["shard"](self)
    finally:
        _S.in_shard = None


def _get_shard(tensor, rank, world_size):
    shard, numel_to_pad = _S.originals["_get_shard"](tensor, rank, world_size)
    handle = _S.in_shard
    if handle is None or not SymmBufferRegistry.is_initialized():
        return shard, numel_to_pad
    reg = SymmBufferRegistry.get_instance()
    if shard.device.type != reg.heap.device.type:
        raise AssertionError("construct FSDP with the module already on the compute device (device_id=...)")
    index = _S.next_index
    _S.next_index += 1
    key = f"fsdp1_flat_{index}"
    buf = reg.allocate_symm_buffer(key, shard.shape, shard.dtype)  # collective: every rank wraps in the same order
    buf.copy_(shard)
    handle._odc_index = index
    handle._odc_key = key
    return buf, numel_to_pad


def _handles(fsdp_model) -> List[FlatParamHandle]:
    return [h for h in _tu._get_fsdp_handles(fsdp_model) if hasattr(h, "_odc_key")]


def _replica(handle: FlatParamHandle) -> Optional[torch.Tensor]:
    return getattr(handle, "_odc_replica", None)


# ------------------------------------------------------------------------------------------
# unshard = gather
# ------------------------------------------------------------------------------------------
def _use_low_precision_shard(self: FlatParamHandle):
    if hasattr(self, "_odc_key"):
        return  # the compute-precision copy lives in the heap and is refreshed once per minibatch
    return _S.originals["_use_low_precision_shard"](self)


def _free_low_precision_sharded_param(self: FlatParamHandle):
    if hasattr(self, "_odc_key"):
        return
    return _S.originals["_free_low_precision_sharded_param"](self)


@torch.no_grad()
def _all_gather_flat_param(self: FlatParamHandle, padded_unsharded_flat_param: torch.Tensor) -> torch.Tensor:
    if not hasattr(self, "_odc_key") or self._use_fake_all_gather:
        return _S.originals["_all_gather_flat_param"](self, padded_unsharded_flat_param)
    _, gather = _services()
    shard = self.flat_param._local_shard if hasattr(self.flat_param, "_local_shard") else self.flat_param.data
    src = shard
    rep = _replica(self)
    if rep is not None and padded_unsharded_flat_param.dtype == rep.dtype:
        src = rep
    if padded_unsharded_flat_param.numel() != src.numel() * self.world_size:
        raise AssertionError(f"expected {src.numel() * self.world_size} elements, got {padded_unsharded_flat_param.numel()}")
    gather.gather_into_tensor(padded_unsharded_flat_param, src, self.process_group)
    return padded_unsharded_flat_param


# ------------------------------------------------------------------------------------------
# reduce = scatter_accumulate
# ------------------------------------------------------------------------------------------
@torch.no_grad()
def _reduce_grad(state: _FSDPState, handle: FlatParamHandle) -> None:
    if not hasattr(handle, "_odc_key"):
        return _S.originals["_reduce_grad"](state, handle)
    if state._comm_hook is not None:
        raise AssertionError("on-demand FSDP1 does not support communication hooks")
    reduction, _ = _services()
    flat_param = handle.flat_param
    unsharded_grad = flat_param.grad.data
    flat_param.grad = None
    factor = float(state._gradient_predivide_factor) * float(state._gradient_postdivide_factor)
    world = state.world_size
    flat = unsharded_grad.reshape(-1)
    shard = (flat.numel() + world - 1) // world      # FSDP1's shard size: the first chunk of ``chunk(world)``
    if not reduction.has_accumulation(handle._odc_key):
        reduction.register(handle._odc_key, shard, flat.dtype, state.process_group)
    done = False
    if shard * world != flat.numel() and config.reduce_from_segments() and flat.is_contiguous():
        # A flat gradient that does not divide by the group size: the last owners' pieces are short or empty.  Stock
        # FSDP1 pads with a full-size copy first; the segmented reduction reads the ragged pieces in place.
        done = reduction.scatter_accumulate_segments(handle._odc_key, [flat], [shard], [0], state.process_group,
                                                     scale=1.0 / factor)
    if not done:
        if shard * world != flat.numel():
            flat = F.pad(flat, [0, shard * world - flat.numel()])
        reduction.scatter_accumulate(handle._odc_key, flat, state.process_group, scale=1.0 / factor)
    _S.touched.add(handle._odc_key)
    # marks "a gradient was produced" for stock bookkeeping; the real value is assigned in pre_optimizer_step
    flat_param._saved_grad_shard = reduction.get_accumulation(handle._odc_key)


def _low_precision_hook_enabled(state: _FSDPState) -> bool:
    """Tell stock FSDP not to widen the unsharded gradient before ``_reduce_grad``.

    Stock FSDP1 casts the whole unsharded gradient to the reduce dtype first (a full-size extra pass).  The
    accumulators here already have the reduce dtype and the reduction widens each element as it adds it, which
    gives the same sums, so for bf16 gradients reduced in fp32 that cast is skipped.
    """
    h = getattr(state, "_handle", None)
    if (h is not None and hasattr(h, "_odc_key") and state._comm_hook is None
            and getattr(h, "_fwd_bwd_param_dtype", None) == torch.bfloat16
            and getattr(h, "_reduce_dtype", None) == torch.float32):
        return True
    return _S.originals["_low_precision_hook_enabled"](state)


def _prepare_gradient_for_optim(self: FlatParamHandle):
    if not hasattr(self, "_odc_key"):
        return _S.originals["prepare_gradient_for_optim"](self)
    if hasattr(self.flat_param, "_saved_grad_shard"):
        delattr(self.flat_param, "_saved_grad_shard")  # never hand the live accumulator to the optimizer


# ------------------------------------------------------------------------------------------
# minibatch boundary
# ------------------------------------------------------------------------------------------
def _device_sync():
    if torch.cuda.is_available():
        torch.cuda.current_stream().synchronize()


@torch.no_grad()
def pre_minibatch_start(fsdp_model) -> None:
    """Zero accumulators, publish updated shards (and their compute-precision copies); collective."""
    _require_patched()
    reduction, _ = _services()
    reg = SymmBufferRegistry.get_instance()
    with nvtx_range("odc::pre_minibatch_start"):
        for h in _handles(fsdp_model):
            shard = h.flat_param._local_shard if hasattr(h.flat_param, "_local_shard") else h.flat_param.data
            if not reduction.has_accumulation(h._odc_key):
                acc_dtype = h._reduce_dtype if getattr(h, "_reduce_dtype", None) is not None else shard.dtype
                if h._uses_param_mixed_precision and getattr(h, "_reduce_dtype", None) is None:
                    acc_dtype = h._fwd_bwd_param_dtype
                reduction.register(h._odc_key, shard.numel(), acc_dtype, h.process_group)
            if h._uses_param_mixed_precision and h._fwd_bwd_param_dtype != shard.dtype:
                if _replica(h) is None:
                    h._odc_replica = reg.allocate_symm_buffer(f"fsdp_params_lowp_{h._odc_key}", shard.shape,
                                                              h._fwd_bwd_param_dtype)
                if getattr(h, "_odc_replica_fresh", False):
                    h._odc_replica_fresh = False      # FusedAdamW wrote the compute-precision copy itself
                else:
                    h._odc_replica.copy_(shard)
        reduction.clear_accumulations()
        _device_sync()
        control.host_barrier()


@torch.no_grad()
def pre_optimizer_step(fsdp_model, materialize_grads: bool = True) -> None:
    """Wait for every contribution (collective) and expose the summed gradient as ``flat_param.grad``.

    ``materialize_grads=False`` leaves ``.grad`` alone: :class:`FusedAdamW` reads the accumulators directly.
    """
    _require_patched()
    if not isinstance(fsdp_model, _FSDPState):
        raise AssertionError("pass the root FSDP module")
    reduction, _ = _services()
    # flat parameters that no rank produced a gradient for keep ``.grad is None``, as under stock FSDP
    used = set()
    for other in reduction.sync(payload=sorted(_S.touched, key=str)):
        used.update(other or ())
    _S.touched = set()
    _S.used = used
    if not materialize_grads:
        return
    for h in _handles(fsdp_model):
        if not reduction.has_accumulation(h._odc_key) or h._odc_key not in used:
            continue
        acc = reduction.get_accumulation(h._odc_key)
        fp = h.flat_param
        shard = fp._local_shard if hasattr(fp, "_local_shard") else fp.data
        # Same dtype: the optimizer reads (and a clip may scale) the accumulator itself.  Nothing adds into it
        # between this synchronisation and the barrier of the next pre_minibatch_start, which clears it anyway.
        g = acc.to(shard.dtype)
        if fp.data.data_ptr() != shard.data_ptr():
            fp.data = shard  # the optimizer must see the sharded flat parameter
        fp.grad = g.view_as(shard)


# ------------------------------------------------------------------------------------------
class FusedAdamW:
    """AdamW over the flat shards, read straight from the accumulators (FSDP1 counterpart of ``fsdp2.FusedAdamW``).

    The reference steps ``torch.optim.AdamW`` over flat parameters whose ``.grad`` is a cast of the accumulator
    (odc/fsdp/fsdp1.py:317-335, examples/llm_training/torch_fsdp.py).  Here one kernel per flat parameter reads
    the summed gradient from its accumulator (the clipping scale folded in), updates the fp32 shard and the
    moments, and writes the compute-precision copy that the peers gather in the next minibatch, so no ``.grad``
    and no separate cast pass exist.  Use with ``pre_optimizer_step(model, materialize_grads=False)``; flat
    parameters that no rank produced a gradient for are skipped, as ``torch.optim.AdamW`` skips ``grad is None``.
    """

    def __init__(self, fsdp_model, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01):
        self.model, self.lr, self.betas, self.eps, self.weight_decay = fsdp_model, lr, betas, eps, weight_decay
        self.state: Dict[str, Dict[str, Any]] = {}    # heap key of the flat parameter -> {"step", "m", "v"}
        self._clip_scale = 1.0

    def _live(self):
        """``(handle, fp32 shard, accumulator)`` of every flat parameter that received a gradient."""
        reduction, _ = _services()
        out = []
        for h in _handles(self.model):
            if h._odc_key not in _S.used or not reduction.has_accumulation(h._odc_key):
                continue
            fp = h.flat_param
            shard = fp._local_shard if hasattr(fp, "_local_shard") else fp.data
            acc = reduction.get_accumulation(h._odc_key)
            if shard.dtype != torch.float32 or acc.dtype != torch.float32:
                raise NotImplementedError("FusedAdamW keeps fp32 shards and fp32 accumulators "
                                          "(patch_fsdp1(reduce_dtype=torch.float32))")
            out.append((h, shard.view(-1), acc.view(-1)))
        return out

    @torch.no_grad()
    def clip_grad_norm_(self, max_norm: float) -> torch.Tensor:
        """Global L2 norm of the summed gradient; the clipping scale is applied inside the next ``step``."""
        live = self._live()
        dev = SymmBufferRegistry.get_instance().heap.device
        total = torch.zeros((), dtype=torch.float32, device=dev)
        for _, _, acc in live:
            if acc.is_cuda:
                from .. import _ext
                part = torch.zeros((), dtype=torch.float32, device=dev)
                _ext.load().sumsq(acc, part)
                total += part
            else:
                total += acc.pow(2).sum()
        if control.world_size() > 1:
            torch.distributed.all_reduce(total)   # shards are disjoint across the ranks (FULL_SHARD over all of them)
        norm = total.sqrt()
        self._clip_scale = float(min(1.0, max_norm / (float(norm) + 1e-6)))
        return norm

    @torch.no_grad()
    def step(self) -> None:
        from .. import ops
        for h, shard, acc in self._live():
            st = self.state.get(h._odc_key)
            if st is None:
                st = self.state[h._odc_key] = {"step": 0, "m": torch.zeros_like(shard), "v": torch.zeros_like(shard)}
            st["step"] += 1
            rep = _replica(h)
            ops.fused_adamw_(shard, acc, st["m"], st["v"], None if rep is None else rep.view(-1), self.lr,
                             self.betas[0], self.betas[1], self.eps, self.weight_decay, st["step"], self._clip_scale)
            if rep is not None:
                h._odc_replica_fresh = True
        self._clip_scale = 1.0

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.model.parameters():
            p.grad = None

    def state_dict(self) -> Dict[str, Any]:
        """This rank's moments by heap key (same sharding on load: same model, same number of ranks)."""
        return {"state": {k: {"step": v["step"], "m": v["m"].clone(), "v": v["v"].clone()} for k, v in self.state.items()},
                "hyper": dict(lr=self.lr, betas=self.betas, eps=self.eps, weight_decay=self.weight_decay)}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.state = {k: {"step": v["step"], "m": v["m"].clone(), "v": v["v"].clone()} for k, v in sd["state"].items()}
        for k, v in sd.get("hyper", {}).items():
            setattr(self, k, v)


# ------------------------------------------------------------------------------------------
def _require_patched():
    if not _S.patched:
        raise RuntimeError("call odc_b200.fsdp.fsdp1.patch_fsdp1() first")


def patch_fsdp1(reduce_dtype: Optional[torch.dtype] = None) -> None:
    """Route FSDP1's flat-parameter all-gather and gradient reduce-scatter through the on-demand primitives."""
    if _S.patched:
        return
    _S.reduce_dtype = reduce_dtype
    _S.originals = {
        "shard": FlatParamHandle.shard,
        "_get_shard": FlatParamHandle._get_shard,
        "_all_gather_flat_param": FlatParamHandle._all_gather_flat_param,
        "_use_low_precision_shard": FlatParamHandle._use_low_precision_shard,
        "_free_low_precision_sharded_param": FlatParamHandle._free_low_precision_sharded_param,
        "prepare_gradient_for_optim": FlatParamHandle.prepare_gradient_for_optim,
        "_reduce_grad": _ru._reduce_grad,
        "_low_precision_hook_enabled": _ru._low_precision_hook_enabled,
    }
    FlatParamHandle.shard = _shard
    FlatParamHandle._get_shard = staticmethod(_get_shard)
    FlatParamHandle._all_gather_flat_param = _all_gather_flat_param
    FlatParamHandle._use_low_precision_shard = _use_low_precision_shard
    FlatParamHandle._free_low_precision_sharded_param = _free_low_precision_sharded_param
    FlatParamHandle.prepare_gradient_for_optim = _prepare_gradient_for_optim
    _ru._reduce_grad = _reduce_grad
    _ru._low_precision_hook_enabled = _low_precision_hook_enabled
    _S.patched = True


def unpatch_fsdp1() -> None:
    if not _S.patched:
        return
    o = _S.originals
    FlatParamHandle.shard = o["shard"]
    FlatParamHandle._get_shard = staticmethod(o["_get_shard"])
    FlatParamHandle._all_gather_flat_param = o["_all_gather_flat_param"]
    FlatParamHandle._use_low_precision_shard = o["_use_low_precision_shard"]
    FlatParamHandle._free_low_precision_sharded_param = o["_free_low_precision_sharded_param"]
    FlatParamHandle.prepare_gradient_for_optim = o["prepare_gradient_for_optim"]
    _ru._reduce_grad = o["_reduce_grad"]
    _ru._low_precision_hook_enabled = o["_low_precision_hook_enabled"]
    _S.patched = False
    _S.reduction = _S.gather = None
    _S.next_index = 0
    _S.touched = set()
    _S.used = set()


def stop() -> None:
    """End of training: stop the services and release the symmetric heap (collective)."""
    if _S.reduction is not None:
        _S.reduction.stop()
    unpatch_fsdp1()
    from .. import finalize_distributed
    finalize_distributed()
