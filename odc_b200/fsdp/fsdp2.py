"""On-demand communication for PyTorch FSDP2 (``fully_shard``).

Public API of the reference (odc/fsdp/fsdp2.py): ``patch_fsdp2(enable_hpz)``,
``patch_lazy_init(module)``, ``pre_minibatch_start(model)``, ``pre_optimizer_step(model)``,
``stop()``, ``get_symm_buffer_memory_breakdown()``, ``get_reduction_service()``,
``get_gather_service()``; call order as in its README (README.md:92-124).

How this integration works (it is a different design from the reference's patch set):

* Only three FSDP2 entry points are replaced: ``foreach_all_gather`` and ``foreach_reduce`` in
  the parameter-group module, and (HPZ mode) the post-forward mesh resolver.  Copy-out,
  resharding and activation-checkpoint handling stay stock.
* After ``patch_lazy_init`` a group's sharded parameters are views of ONE flat buffer in the
  symmetric heap (the optimizer updates it in place; DTensor/DCP layout is unchanged).  With
  mixed precision a second flat buffer holds the shards in ``param_dtype``; it is refreshed
  once per minibatch, so ``gather`` moves compute-precision bytes instead of fp32 masters
  (the reference gathers the original dtype and casts afterwards, odc/fsdp/fsdp2.py:339-351).
* ``foreach_reduce`` adds the unsharded gradients into the owners' accumulators: straight from
  the per-parameter tensors in one segmented ``scatter_accumulate`` launch where the transport
  can (no rank-major staging copy), otherwise flattened rank-major first; no gradient is
  attached to a parameter until
  ``pre_optimizer_step``, which waits for the arrivals (the one synchronisation per
  minibatch), applies the divide factor, runs the HSDP replicate-dimension all-reduce once
  per group and assigns ``sharded_param.grad``.  Ranks may run different numbers of
  microbatches, including zero.
* ``reshard_after_forward=int`` with ``enable_hpz``: each rank keeps, in a symmetric buffer, the
  compute-precision shards of ``W/int`` owners (a secondary partition inside a group of
  ``int`` ranks), refreshed once per minibatch; forward and backward unshards then pull only
  from that group (odc/fsdp/fsdp2.py:745-791, 961-1020 describe the reference's variant).
"""
from __future__ import annotations

import logging
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
from torch.distributed.fsdp._fully_shard import _fsdp_collectives, _fsdp_param_group, _fully_shard
from torch.distributed.fsdp._fully_shard._fsdp_collectives import AllGatherResult
from torch.distributed.fsdp._fully_shard._fsdp_common import (DDPMeshInfo, FSDPMeshInfo, _get_dim0_padded_size)
from torch.distributed.fsdp._fully_shard._fsdp_param import FSDPParam, ShardedState
from torch.distributed.fsdp._fully_shard._fsdp_param_group import FSDPParamGroup

from .. import config
from ..primitives import GatherService, ReductionService
from ..runtime import control
from ..runtime.registry import SymmBufferRegistry
from ..utils.nvtx import nvtx_range, nvtx_record_function

logger = logging.getLogger("odc_b200")


@dataclass
class _GroupInfo:
    """Per parameter-group state kept by this integration."""
    index: int
    group: FSDPParamGroup
    key: str
    master: torch.Tensor                      # flat shards, original dtype (symmetric)
    replica: Optional[torch.Tensor]           # flat shards, param_dtype (symmetric) or None
    numels: List[int]                         # padded shard numel per fsdp_param
    trainable: List[int]                      # indices of params with requires_grad
    acc_numel: int
    acc_offsets: Dict[int, int]               # id(fsdp_param) -> offset in the accumulator
    hpz_size: int = 0
    hpz: Optional[torch.Tensor] = None        # [W/hpz_size * S] in compute dtype (symmetric)
    hpz_ranks: List[int] = field(default_factory=list)
    reduce_calls: int = 0
    divide: Dict[str, Any] = field(default_factory=dict)
    replica_fresh: bool = False               # the optimizer already wrote the low-precision copy
    position: Dict[int, int] = field(default_factory=dict)   # id(fsdp_param) -> index in the group
    offsets: List[int] = field(default_factory=list)         # element offset of each fsdp_param in the flat buffers
    touched: set = field(default_factory=set)  # parameters this rank reduced a gradient for in this minibatch
    used: Optional[set] = None                 # union of `touched` over all ranks (None: not known, treat as all)

    @property
    def acc_key(self) -> str:
        return f"{self.index}"


class _State:
    patched = False
    enable_hpz = False
    originals: Dict[str, Any] = {}
    reduction: Optional[ReductionService] = None
    gather: Optional[GatherService] = None
    infos: List[_GroupInfo] = []
    by_param: Dict[int, _GroupInfo] = {}
    pending_hpz: Optional[int] = None
    next_index = 0


_S = _State


def get_reduction_service() -> Optional[ReductionService]:
    return _S.reduction


def get_gather_service() -> Optional[GatherService]:
    return _S.gather


def get_fsdp_params_key(index: int) -> str:
    return f"fsdp_params_gather_{index}"


def get_hpz_params_key(key: str) -> str:
    return f"hpz_{key}"


def get_replica_key(key: str) -> str:
    return f"fsdp_params_lowp_{key}"


# ------------------------------------------------------------------------------------------
# lazy init: move a group's shards into the symmetric heap
# ------------------------------------------------------------------------------------------
@torch.no_grad()
def patch_lazy_init(fsdp_module) -> None:
    """Arrange for ``fsdp_module``'s parameter group to live in the symmetric heap.

    Call for EVERY module that was ``fully_shard``-ed, after any checkpoint load and before the
    first forward.  The move happens right after the group's stock lazy init.
    """
    _require_patched()
    state = fsdp_module._get_fsdp_state()
    group = state._fsdp_param_group
    if group is None or getattr(group, "_odc_lazy_patched", False):
        return
    stock = group.lazy_init
    index = _S.next_index
    _S.next_index += 1

    def lazy_init_then_pin():
        stock()
        if getattr(group, "_odc_info", None) is None:
            _pin_group(group, index)

    group.lazy_init = lazy_init_then_pin
    group._odc_lazy_patched = True


def _supported(group: FSDPParamGroup) -> Optional[str]:
    if not isinstance(group.mesh_info, FSDPMeshInfo):
        return "not sharded (replicate-only mesh)"
    for p in group.fsdp_params:
        if p.offload_to_cpu:
            return "CPU offload"
        if p.is_dtensor:
            return "tensor-parallel (DTensor) parameters"
        if hasattr(p._sharded_local_tensor, "fsdp_pre_all_gather"):
            return "tensor-subclass all-gather extensions"
    dtypes = {p._sharded_param_data.dtype for p in group.fsdp_params}
    if len(dtypes) != 1:
        return f"mixed original dtypes {dtypes}"
    pd = {p.param_dtype for p in group.fsdp_params}
    if len(pd) != 1:
        return f"mixed param dtypes {pd}"
    return None


@torch.no_grad()
def _pin_group(group: FSDPParamGroup, index: int) -> None:
    why = _supported(group)
    if why is not None:
        raise NotImplementedError(f"on-demand FSDP2 does not support {why} (group {group._module_fqn})")
    registry = SymmBufferRegistry.get_instance()
    params = group.fsdp_params
    numels = [p._sharded_param_data.numel() for p in params]
    total = sum(numels)
    orig_dtype = params[0]._sharded_param_data.dtype
    key = get_fsdp_params_key(index)
    master = registry.allocate_symm_buffer(key, (total,), orig_dtype)
    _bind_params_to(master, params, numels, copy=True)
    param_dtype = params[0].param_dtype
    replica = None
    if param_dtype is not None and param_dtype != orig_dtype:
        replica = registry.allocate_symm_buffer(get_replica_key(key), (total,), param_dtype)
        replica.copy_(master)
    trainable = [i for i, p in enumerate(params) if p.sharded_param.requires_grad]
    offs, o = {}, 0
    for i in trainable:
        offs[id(params[i])] = o
        o += numels[i]
    info = _GroupInfo(index, group, key, master, replica, numels, trainable, o, offs)
    info.position = {id(p): i for i, p in enumerate(params)}
    info.offsets = [sum(numels[:i]) for i in range(len(numels))]
    hpz = getattr(group, "_odc_hpz_size", 0)
    if _S.enable_hpz and hpz:
        ranks = control.group_ranks(group.mesh_info.shard_process_group)
        W = len(ranks)
        if W % hpz != 0:
            raise ValueError(f"reshard_after_forward={hpz} must divide the shard group size {W}")
        me = ranks.index(control.rank())
        base = me - me % hpz
        info.hpz_size = hpz
        info.hpz_ranks = ranks[base:base + hpz]
        info.hpz = registry.allocate_symm_buffer(get_hpz_params_key(key), ((W // hpz) * total,),
                                                 param_dtype or orig_dtype)
    if o > 0:
        reduce_dtype = group._reduce_dtype or param_dtype or orig_dtype
        _S.reduction.register(info.acc_key, o, reduce_dtype, group.mesh_info.shard_process_group)
    group._odc_info = info
    _S.infos.append(info)
    for p in params:
        _S.by_param[id(p)] = info


def _bind_params_to(flat: torch.Tensor, params: List[FSDPParam], numels: List[int], copy: bool) -> None:
    off = 0
    for p, n in zip(params, numels):
        view = flat[off:off + n]
        if copy:
            view.copy_(p._sharded_param_data)
        p._sharded_param_data = view
        padded = view.view(p.padded_sharded_param_size)
        dim = p.fsdp_placement.dim
        local = p.sharded_param._local_tensor
        length = local.size(dim) if local.numel() > 0 else 0
        p.sharded_param._local_tensor = padded.narrow(dim, 0, length)
        off += n


@torch.no_grad()
def repin_sharded_params(model) -> None:
    """Re-attach parameters to the heap after ``load_state_dict(assign=True)`` replaced them.

    Stock ``reset_sharded_param`` re-derives the flat shard from whatever tensor the module now
    holds, which silently detaches it from the symmetric buffer peers read from.
    """
    for info in _infos_of(model):
        for p in info.group.fsdp_params:
            p.reset_sharded_param()
        _bind_params_to(info.master, info.group.fsdp_params, info.numels, copy=True)


# ------------------------------------------------------------------------------------------
# unshard = gather
# ------------------------------------------------------------------------------------------
@torch.no_grad()
def _odc_foreach_all_gather(fsdp_params, group, async_op, all_gather_copy_in_stream, all_gather_stream,
                            device, all_gather_comm):
    info = _S.by_param.get(id(fsdp_params[0])) if fsdp_params else None
    if (info is None or len(fsdp_params) != len(info.numels)
            or any(p.sharded_state != ShardedState.SHARDED for p in fsdp_params)):
        return _S.originals["foreach_all_gather"](fsdp_params, group, async_op, all_gather_copy_in_stream,
                                                  all_gather_stream, device, all_gather_comm)
    world = group.size()
    total = sum(info.numels)
    if info.hpz is not None:
        src, pg_ranks = info.hpz, info.hpz_ranks
    else:
        src, pg_ranks = (info.replica if info.replica is not None else info.master), None
    handle = _fsdp_collectives._get_device_handle(device.type)
    with handle.stream(all_gather_stream):
        out = all_gather_comm.allocate((total * world,), dtype=src.dtype, device=device)
        if pg_ranks is None:
            _S.gather.gather_into_tensor(out, src, group)
        else:
            _S.gather.gather_ranks(out, src, pg_ranks)
        event = all_gather_stream.record_event()
    dtypes = [[src.dtype] for _ in info.numels]
    nums = [[n] for n in info.numels]
    return AllGatherResult(out, event, None, dtypes, nums, list(info.numels))


def _odc_all_gather_inputs(self):
    """Single-rank shard groups: stock FSDP2 skips the all-gather and builds the unsharded parameter from
    ``all_gather_inputs``, casting the fp32 shard to the compute dtype on every unshard.  The group's low-precision
    copy in the heap already holds exactly that (refreshed once per minibatch), so hand out a view of it."""
    info = _S.by_param.get(id(self))
    if (info is not None and info.replica is not None and info.hpz is None
            and self.sharded_state == ShardedState.SHARDED and info.group.mesh_info.shard_mesh_size == 1):
        i = info.position[id(self)]
        off = info.offsets[i]
        return [info.replica[off:off + info.numels[i]]]
    return _S.originals["all_gather_inputs"].fget(self)


# ------------------------------------------------------------------------------------------
# post-backward = scatter_accumulate (no gradient is materialised here)
# ------------------------------------------------------------------------------------------
@torch.no_grad()
def _odc_foreach_reduce(fsdp_params, unsharded_grads, reduce_scatter_group, reduce_scatter_stream,
                        reduce_scatter_comm, orig_dtype, reduce_dtype, device, gradient_divide_factor,
                        all_reduce_group, all_reduce_stream, all_reduce_grads, partial_reduce_output,
                        all_reduce_hook, force_sum_reduction_for_comms=False):
    info = _S.by_param.get(id(fsdp_params[0])) if fsdp_params else None
    if info is None or reduce_scatter_group is None:
        return _S.originals["foreach_reduce"](
            fsdp_params, unsharded_grads, reduce_scatter_group, reduce_scatter_stream, reduce_scatter_comm,
            orig_dtype, reduce_dtype, device, gradient_divide_factor, all_reduce_group, all_reduce_stream,
            all_reduce_grads, partial_reduce_output, all_reduce_hook, force_sum_reduction_for_comms)
    grad_dtypes = {g.dtype for g in unsharded_grads}
    if len(grad_dtypes) != 1:
        raise AssertionError(f"FSDP reduce-scatter expects uniform gradient dtype but got {grad_dtypes}")
    reduce_dtype = reduce_dtype or unsharded_grads[0].dtype
    world = reduce_scatter_group.size()
    handle = _fsdp_collectives._get_device_handle(device.type)
    current = handle.current_stream()
    for i, (p, g) in enumerate(zip(fsdp_params, unsharded_grads)):
        if (dim := p.fsdp_placement.dim) != 0:
            unsharded_grads[i] = torch.cat(torch.chunk(g, world, dim=dim), dim=0)
    grad_dtype = unsharded_grads[0].dtype
    acc_dtype = _S.reduction.get_accumulation(info.acc_key).dtype
    # First choice: reduce straight from the per-parameter gradients.  A dim-0 chunk of a contiguous tensor is
    # contiguous, so no rank-major staging copy is needed; the kernel widens each element as it adds it.
    reduce_scatter_stream.wait_stream(current)
    done = False
    if config.reduce_from_segments() and all(g.is_contiguous() for g in unsharded_grads):
        chunks = [_get_dim0_padded_size(g.size(), world).numel() // world for g in unsharded_grads]
        offsets = [info.acc_offsets[id(p)] for p in fsdp_params]
        with handle.stream(reduce_scatter_stream):
            done = _S.reduction.scatter_accumulate_segments(info.acc_key, unsharded_grads, chunks, offsets,
                                                            reduce_scatter_group)
            if done:
                event = reduce_scatter_stream.record_event()
        if done:
            # FSDP keeps the returned tensor until it has waited for the event; it carries the gradients along so
            # that their memory is not reused while the kernel may still read it
            rs_input = torch.empty(0, dtype=grad_dtype, device=device)
            rs_input._odc_keepalive = list(unsharded_grads)
            unsharded_grads.clear()
    if not done:
        # Flattened path.  Stock FSDP2 widens the gradients to the reduce dtype while flattening them; the
        # accumulators already have the reduce dtype and the transport widens while adding, which gives the same
        # sums, so the staging copy keeps the (narrower) gradient dtype.
        stage_dtype = reduce_dtype
        if acc_dtype == reduce_dtype == torch.float32 and grad_dtype == torch.bfloat16:
            stage_dtype = grad_dtype
        rs_input = reduce_scatter_comm.allocate((info.acc_numel * world,), dtype=stage_dtype, device=device)
        rs2d = rs_input.view(world, info.acc_numel)
        all_present = len(fsdp_params) == len(info.trainable)
        if all_present:
            torch.ops.fsdp.chunk_cat(unsharded_grads, dim=0, num_chunks=world, out=rs2d)
        else:  # some parameters received no gradient in this backward: their columns contribute zero
            rs2d.zero_()
            for p, g in zip(fsdp_params, unsharded_grads):
                o = info.acc_offsets[id(p)]
                n = _get_dim0_padded_size(g.size(), world).numel() // world
                torch.ops.fsdp.chunk_cat([g], dim=0, num_chunks=world, out=rs2d[:, o:o + n])
        unsharded_grads.clear()
        reduce_scatter_stream.wait_stream(current)
        with handle.stream(reduce_scatter_stream):
            _S.reduction.scatter_accumulate(info.acc_key, rs_input, reduce_scatter_group)
            event = reduce_scatter_stream.record_event()
    info.reduce_calls += 1
    info.touched.update(info.position[id(p)] for p in fsdp_params)
    info.divide = dict(factor=gradient_divide_factor, all_reduce_group=all_reduce_group,
                       all_reduce_hook=all_reduce_hook, orig_dtype=orig_dtype)
    return rs_input, event, event, None, None, None


# ------------------------------------------------------------------------------------------
# minibatch boundary
# ------------------------------------------------------------------------------------------
def _fsdp_modules(model):
    from torch.distributed.fsdp import FSDPModule
    return [m for m in model.modules() if isinstance(m, FSDPModule)]


def _infos_of(model) -> List[_GroupInfo]:
    out = []
    for m in _fsdp_modules(model):
        g = m._get_fsdp_state()._fsdp_param_group
        info = getattr(g, "_odc_info", None) if g is not None else None
        if info is not None:
            out.append(info)
    return sorted(out, key=lambda i: i.index)


def _device_sync():
    if torch.cuda.is_available():
        torch.cuda.current_stream().synchronize()


@torch.no_grad()
def pre_minibatch_start(model) -> None:
    """Zero the accumulators and publish this rank's freshly updated shards (collective).

    After the barrier inside, every rank may gather any shard at any time until the next
    optimizer step; nothing else synchronises ranks during the minibatch.
    """
    _require_patched()
    state = model._get_fsdp_state()
    if state._is_root is None:
        state._lazy_init()  # allocate and fill the symmetric buffers before any peer can gather them
    infos = _infos_of(model)
    with nvtx_range("odc::pre_minibatch_start"):
        _S.reduction.clear_accumulations()
        for info in infos:
            if info.replica is not None and not info.replica_fresh:
                _copy_to_replica(info)
        _device_sync()
        control.host_barrier()
        hpz = [i for i in infos if i.hpz is not None]
        if hpz:
            for info in hpz:
                _refresh_secondary_shards(info)
            _device_sync()
            control.host_barrier()


def _copy_to_replica(info: _GroupInfo) -> None:
    if info.master.is_cuda and info.master.dtype == torch.float32 and info.replica.dtype == torch.bfloat16:
        from .. import _ext
        _ext.load().cast_f32_to_bf16(info.master, info.replica)
    else:
        info.replica.copy_(info.master)


def _refresh_secondary_shards(info: _GroupInfo) -> None:
    """Pull the shards of the ``W/G`` owners this rank re-serves inside its HPZ group."""
    ranks = control.group_ranks(info.group.mesh_info.shard_process_group)
    W, G = len(ranks), info.hpz_size
    me = ranks.index(control.rank())
    j = me % G                                   # position in the HPZ group = block of owners served
    owners = ranks[j * (W // G):(j + 1) * (W // G)]
    src = info.replica if info.replica is not None else info.master
    _S.gather.gather_ranks(info.hpz, src, owners)


@torch.no_grad()
def pre_optimizer_step(model, materialize_grads: bool = True) -> None:
    """Wait for every contribution to this rank's shards and turn them into ``.grad`` (collective).

    ``materialize_grads=False`` stops after the synchronisation (and the HSDP all-reduce): the
    summed gradients stay in the accumulators, where :class:`FusedAdamW` consumes them directly.
    """
    _require_patched()
    infos = _infos_of(model)
    # which parameters received a gradient from ANY rank: the others keep ``.grad is None`` (as under stock FSDP,
    # where an optimizer skips them) instead of taking a step on an all-zero gradient
    mine = {info.index: sorted(info.touched) for info in infos}
    everyone = _S.reduction.sync(payload=mine)
    for info in infos:
        info.used = set()
        for other in everyone:
            info.used.update((other or {}).get(info.index, ()))
        info.touched = set()
    for info in infos:
        with nvtx_range(f"odc::update_gradients:{info.group._module_fqn}"):
            if materialize_grads:
                _update_gradients(info)
            else:
                _reduce_replicas_in_place(info)
    for info in infos:
        info.replica_fresh = False


def _divide_factor(info: _GroupInfo) -> float:
    group = info.group
    mesh_info = group.mesh_info
    replicate_pg = mesh_info.replicate_process_group if isinstance(mesh_info, DDPMeshInfo) else None
    dp = mesh_info.shard_mesh_size * (replicate_pg.size() if replicate_pg is not None else 1)
    return group.gradient_divide_factor if group.gradient_divide_factor is not None else float(dp)


def _reduce_replicas_in_place(info: _GroupInfo) -> None:
    if info.acc_numel == 0:
        return
    mesh_info = info.group.mesh_info
    if isinstance(mesh_info, DDPMeshInfo) and info.group.all_reduce_grads:
        acc = _S.reduction.get_accumulation(info.acc_key)
        dist.all_reduce(acc, group=mesh_info.replicate_process_group, op=dist.ReduceOp.SUM)


def transport_launches() -> int:
    """Kernels launched by the communication services so far (benchmark accounting)."""
    n = 0
    for svc in (_S.gather, _S.reduction):
        if svc is not None:
            n += getattr(svc.transport, "launches", 0)
    return n


def _update_gradients(info: _GroupInfo) -> None:
    group = info.group
    if info.acc_numel == 0:
        return
    acc = _S.reduction.get_accumulation(info.acc_key)
    mesh_info = group.mesh_info
    shard_size = mesh_info.shard_mesh_size
    replicate_pg = mesh_info.replicate_process_group if isinstance(mesh_info, DDPMeshInfo) else None
    dp = shard_size * (replicate_pg.size() if replicate_pg is not None else 1)
    factor = group.gradient_divide_factor if group.gradient_divide_factor is not None else float(dp)
    out = acc / factor if factor != 1 else acc.clone()
    if replicate_pg is not None and group.all_reduce_grads:
        dist.all_reduce(out, group=replicate_pg, op=dist.ReduceOp.SUM)
    if group._all_reduce_hook is not None:
        group._all_reduce_hook(out)
    orig_dtype = group._orig_dtype
    if orig_dtype is not None and out.dtype != orig_dtype:
        out = out.to(orig_dtype)
    for i in info.trainable:
        if info.used is not None and i not in info.used:
            continue  # no rank produced a gradient for this parameter in this minibatch
        p = group.fsdp_params[i]
        o = info.acc_offsets[id(p)]
        new_grad = torch.as_strided(out, size=p.sharded_size, stride=p.contiguous_sharded_stride, storage_offset=o)
        if p.sharded_param.grad is not None:
            p.sharded_param.grad._local_tensor += new_grad
        else:
            p.sharded_param.grad = p.to_sharded_dtensor(new_grad)
        for hook in (getattr(p.sharded_param, "_post_accumulate_grad_hooks", {}) or {}).values():
            hook(p.sharded_param)
    info.reduce_calls = 0


# ------------------------------------------------------------------------------------------
# HPZ: keep `reshard_after_forward=int` as "secondary partition size"
# ------------------------------------------------------------------------------------------
def _hpz_get_post_forward_mesh_info(reshard_after_forward, mesh_info):
    stock = _S.originals["_get_post_forward_mesh_info"]
    if (_S.enable_hpz and not isinstance(reshard_after_forward, bool) and isinstance(reshard_after_forward, int)
            and reshard_after_forward >= 1):
        if mesh_info.shard_mesh_size % reshard_after_forward != 0:
            raise ValueError(f"reshard_after_forward={reshard_after_forward} must divide the shard mesh size "
                             f"{mesh_info.shard_mesh_size}")
        _S.pending_hpz = int(reshard_after_forward)
        return stock(True, mesh_info)  # stock state machine: fully reshard after forward
    _S.pending_hpz = None
    return stock(reshard_after_forward, mesh_info)


def _hpz_init_param_group(state, *args, **kwargs):
    _S.originals["_init_param_group"](state, *args, **kwargs)
    if _S.pending_hpz and getattr(state, "_fsdp_param_group", None) is not None:
        state._fsdp_param_group._odc_hpz_size = _S.pending_hpz
    _S.pending_hpz = None


# ------------------------------------------------------------------------------------------
# patch / stop
# ------------------------------------------------------------------------------------------
def _require_patched():
    if not _S.patched:
        raise RuntimeError("call odc_b200.fsdp.fsdp2.patch_fsdp2() first")


def patch_fsdp2(enable_hpz: bool = False) -> None:
    """Route FSDP2's unshard and gradient reduction through the on-demand primitives.

    May be called again only with the same ``enable_hpz`` (odc/fsdp/fsdp2.py:1109-1115).
    Requires ``init_nvshmem()`` to have been called.
    """
    if _S.patched:
        if _S.enable_hpz != enable_hpz:
            raise RuntimeError("patch_fsdp2 was already applied with a different enable_hpz")
        return
    _S.enable_hpz = enable_hpz
    _S.reduction = ReductionService()
    _S.gather = GatherService()
    _S.originals = {
        "foreach_all_gather": _fsdp_param_group.foreach_all_gather,
        "foreach_reduce": _fsdp_param_group.foreach_reduce,
        "record_function": _fsdp_param_group.record_function,
        "_get_post_forward_mesh_info": _fully_shard._get_post_forward_mesh_info,
        "_init_param_group": _fully_shard._init_param_group,
        "all_gather_inputs": FSDPParam.all_gather_inputs,
    }
    _fsdp_param_group.foreach_all_gather = _odc_foreach_all_gather
    _fsdp_param_group.foreach_reduce = _odc_foreach_reduce
    _fsdp_param_group.record_function = nvtx_record_function
    _fully_shard._get_post_forward_mesh_info = _hpz_get_post_forward_mesh_info
    _fully_shard._init_param_group = _hpz_init_param_group
    FSDPParam.all_gather_inputs = property(_odc_all_gather_inputs)
    _S.patched = True


def unpatch_fsdp2() -> None:
    if not _S.patched:
        return
    _fsdp_param_group.foreach_all_gather = _S.originals["foreach_all_gather"]
    _fsdp_param_group.foreach_reduce = _S.originals["foreach_reduce"]
    _fsdp_param_group.record_function = _S.originals["record_function"]
    _fully_shard._get_post_forward_mesh_info = _S.originals["_get_post_forward_mesh_info"]
    _fully_shard._init_param_group = _S.originals["_init_param_group"]
    FSDPParam.all_gather_inputs = _S.originals["all_gather_inputs"]
    _S.patched = False
    _S.infos, _S.by_param, _S.next_index, _S.pending_hpz = [], {}, 0, None
    _S.reduction = _S.gather = None


def stop() -> None:
    """End of training: stop the services and release the symmetric heap (collective).

    Parameters are views of heap memory, so the model must not be used afterwards.
    """
    if _S.reduction is not None:
        _S.reduction.stop()
    unpatch_fsdp2()
    from .. import finalize_distributed
    finalize_distributed()


def get_symm_buffer_memory_breakdown() -> Dict[str, float]:
    """GiB of symmetric memory per purpose (odc/fsdp/fsdp2.py:1147-1172)."""
    out = {"fsdp_params": 0.0, "accumulation": 0.0, "lowp_replica": 0.0, "hpz_buffer": 0.0, "other": 0.0}
    if not SymmBufferRegistry.is_initialized():
        return out
    for key, nbytes in SymmBufferRegistry.get_instance().memory_by_key().items():
        k = str(key)
        gib = nbytes / 2**30
        if k.startswith("hpz_"):
            out["hpz_buffer"] += gib
        elif k.startswith("fsdp_params_lowp_"):
            out["lowp_replica"] += gib
        elif k.startswith("fsdp_params"):
            out["fsdp_params"] += gib
        elif k.startswith("rs_accumulation"):
            out["accumulation"] += gib
        else:
            out["other"] += gib
    out["total"] = sum(out.values())
    return out


# ------------------------------------------------------------------------------------------
# optimizer on the flat shards
# ------------------------------------------------------------------------------------------
def _used_ranges(info: _GroupInfo, steps: List[int]):
    """``(start, stop, step)`` element ranges of the group's flat shard whose parameters received a gradient.

    ``steps[i]`` is the number of updates parameter i has had including this one; adjacent parameters with the same
    count are merged (the usual case is one range for the whole group).
    """
    ranges, start = [], 0
    for i, n in enumerate(info.numels):
        if n and (info.used is None or i in info.used):
            if ranges and ranges[-1][1] == start and ranges[-1][2] == steps[i]:
                ranges[-1] = (ranges[-1][0], start + n, steps[i])
            else:
                ranges.append((start, start + n, steps[i]))
        start += n
    return ranges


class FusedAdamW:
    """AdamW that runs once per parameter group directly on the flat symmetric shard.

    The reference steps ``torch.optim.AdamW`` over DTensor shards that alias symmetric memory
    (examples/llm_training/torch_fsdp2.py:322).  Here one kernel per group reads the summed
    gradient straight from the accumulator (folding the divide factor and the clipping scale),
    updates the fp32 master shard and moments, and writes the compute-precision copy that peers
    gather, so no ``.grad`` tensor and no separate cast pass exist.  Use with
    ``pre_optimizer_step(model, materialize_grads=False)``.
    """

    def __init__(self, model, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.01):
        self.model, self.lr, self.betas, self.eps, self.weight_decay = model, lr, betas, eps, weight_decay
        self.step_count = 0
        self.state: Dict[int, Dict[str, torch.Tensor]] = {}
        self.param_steps: Dict[int, List[int]] = {}   # group index -> updates applied to each of its parameters
        self._clip_scale = 1.0

    def _groups(self) -> List[_GroupInfo]:
        infos = _infos_of(self.model)
        for info in infos:
            if len(info.trainable) != len(info.numels):
                raise NotImplementedError("FusedAdamW needs every parameter of a group to be trainable")
            if info.master.dtype != torch.float32:
                raise NotImplementedError("FusedAdamW keeps fp32 master shards")
        return infos

    @torch.no_grad()
    def clip_grad_norm_(self, max_norm: float) -> torch.Tensor:
        """Global L2 norm of the averaged gradient; the clipping scale is applied inside the next ``step``."""
        infos = self._groups()
        dev = infos[0].master.device
        total = torch.zeros((), dtype=torch.float32, device=dev)
        for info in infos:
            acc = _S.reduction.get_accumulation(info.acc_key)
            f = 1.0 / _divide_factor(info)
            if acc.is_cuda:
                from .. import _ext
                part = torch.zeros((), dtype=torch.float32, device=dev)
                _ext.load().sumsq(acc, part)
                total += part * (f * f)
            else:
                total += (acc.float() * f).pow(2).sum()
        if dist.is_initialized() and dist.get_world_size() > 1:
            # shards of one group are disjoint across its shard group; replicas hold identical sums
            rep = 1
            mi = infos[0].group.mesh_info
            if isinstance(mi, DDPMeshInfo):
                rep = mi.replicate_process_group.size()
            dist.all_reduce(total)
            total = total / rep
        norm = total.sqrt()
        self._clip_scale = float(min(1.0, max_norm / (float(norm) + 1e-6)))
        return norm

    @torch.no_grad()
    def step(self) -> None:
        from .. import ops
        self.step_count += 1
        for info in self._groups():
            acc = _S.reduction.get_accumulation(info.acc_key)
            st = self.state.get(info.index)
            if st is None:
                st = {"m": torch.zeros_like(info.master), "v": torch.zeros_like(info.master)}
                self.state[info.index] = st
            # bias correction counts the updates a parameter has actually had (one that no rank used is skipped)
            steps = self.param_steps.setdefault(info.index, [self.step_count - 1] * len(info.numels))
            for i in range(len(steps)):
                if info.used is None or i in info.used:
                    steps[i] += 1
            for a, b, t in _used_ranges(info, steps):
                ops.fused_adamw_(info.master[a:b], acc[a:b], st["m"][a:b], st["v"][a:b],
                                 None if info.replica is None else info.replica[a:b], self.lr, self.betas[0],
                                 self.betas[1], self.eps, self.weight_decay, t,
                                 self._clip_scale / _divide_factor(info))
            info.replica_fresh = info.replica is not None
        self._clip_scale = 1.0

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.model.parameters():
            p.grad = None

    def state_dict(self) -> Dict[str, Any]:
        return {"step": self.step_count, "state": {k: {n: t.clone() for n, t in v.items()} for k, v in self.state.items()},
                "param_steps": {k: list(v) for k, v in self.param_steps.items()},
                "hyper": dict(lr=self.lr, betas=self.betas, eps=self.eps, weight_decay=self.weight_decay)}

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        self.step_count = sd["step"]
        self.state = {k: {n: t.clone() for n, t in v.items()} for k, v in sd["state"].items()}
        self.param_steps = {k: list(v) for k, v in sd.get("param_steps", {}).items()}
        for k, v in sd.get("hyper", {}).items():
            setattr(self, k, v)

    # -- the layout ``torch.optim.AdamW`` has under FSDP2, so checkpoints move between the two ------------------
    def _param_slots(self):
        """``(name, info, index in group, fsdp_param, element offset in the flat shard)`` in model order."""
        root = self.model._get_fsdp_state()
        if root._is_root is None:
            root._lazy_init()  # moves the shards into the heap and creates the per-group records used below
        names = {id(prm): n for n, prm in self.model.named_parameters()}
        order = {n: k for k, n in enumerate(names.values())}
        slots = []
        for info in self._groups():
            off = 0
            for i, p in enumerate(info.group.fsdp_params):
                slots.append((names[id(p.sharded_param)], info, i, p, off))
                off += info.numels[i]
        return sorted(slots, key=lambda slot: order[slot[0]])

    def _moments(self, info: _GroupInfo) -> Dict[str, torch.Tensor]:
        st = self.state.get(info.index)
        if st is None:
            st = self.state[info.index] = {"m": torch.zeros_like(info.master), "v": torch.zeros_like(info.master)}
        return st

    @torch.no_grad()
    def full_state_dict(self) -> Dict[str, Any]:
        """Unsharded state keyed by parameter name, in the format of a full ``AdamW`` state dict (collective).

        It is what ``get_optimizer_state_dict(..., full_state_dict=True)`` returns for ``torch.optim.AdamW`` on the
        same model — ``step`` / ``exp_avg`` / ``exp_avg_sq`` per parameter plus one parameter group — so a run can
        be resumed with either optimizer, under either engine.
        """
        state = {}
        for name, info, i, p, off in self._param_slots():
            st = self._moments(info)
            steps = self.param_steps.get(info.index, [self.step_count] * len(info.numels))
            entry = {"step": torch.tensor(float(steps[i]))}
            for key, flat in (("exp_avg", st["m"]), ("exp_avg_sq", st["v"])):
                local = torch.as_strided(flat, p.sharded_size, p.contiguous_sharded_stride, off)
                entry[key] = p.to_sharded_dtensor(local).full_tensor().cpu()
            state[name] = entry
        probe = torch.optim.AdamW([torch.zeros(1, requires_grad=True)], lr=self.lr, betas=tuple(self.betas),
                                  eps=self.eps, weight_decay=self.weight_decay)
        group = dict(probe.state_dict()["param_groups"][0])
        group["params"] = list(state.keys())
        return {"state": state, "param_groups": [group]}

    @torch.no_grad()
    def load_full_state_dict(self, sd: Dict[str, Any]) -> None:
        """Inverse of :meth:`full_state_dict`; also takes what stock FSDP2 + ``torch.optim.AdamW`` saved (collective)."""
        from torch.distributed.tensor import DTensor, distribute_tensor
        steps = []
        for name, info, i, p, off in self._param_slots():
            st = self._moments(info)
            per_param = self.param_steps.setdefault(info.index, [0] * len(info.numels))
            entry = sd["state"].get(name)
            if entry is None:  # a parameter that had not been updated yet when the checkpoint was written
                per_param[i] = 0
                continue
            ref = p.sharded_param
            for key, flat in (("exp_avg", st["m"]), ("exp_avg_sq", st["v"])):
                src = entry[key]
                if not isinstance(src, DTensor):
                    src = distribute_tensor(src.to(device=flat.device, dtype=flat.dtype), ref.device_mesh, ref.placements)
                torch.as_strided(flat, p.sharded_size, p.contiguous_sharded_stride, off).copy_(src.to_local())
            per_param[i] = int(float(entry["step"]))
            steps.append(per_param[i])
        self.step_count = max(steps, default=0)
        if sd.get("param_groups"):
            g = sd["param_groups"][0]
            self.lr, self.betas, self.eps = g.get("lr", self.lr), tuple(g.get("betas", self.betas)), g.get("eps", self.eps)
            self.weight_decay = g.get("weight_decay", self.weight_decay)
