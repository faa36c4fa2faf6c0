"""Host-side control plane: process-group helpers and the comm stream.

The data plane never needs the peer's *process* to take part; the control plane is the
handful of host collectives that remain (heap bootstrap, collective allocation, the
once-per-minibatch count exchange).  They run on a gloo group so that they never enqueue
work on, or synchronise with, a CUDA stream.

Reference behaviour covered: odc/primitives/utils.py:175-209 (comm stream, local world
size, per-node groups) and the NCCL object collectives listed at
odc/primitives/scatter_accumulate.py:737-739.
"""
from __future__ import annotations

import os
from typing import Any, List, Optional

import torch
import torch.distributed as dist

from .. import config

_control_pg: Optional[dist.ProcessGroup] = None
_comm_stream = None
_local_world_pg = None
_heartbeat = None


def world_size() -> int:
    return dist.get_world_size() if dist.is_initialized() else 1


def rank() -> int:
    return dist.get_rank() if dist.is_initialized() else 0


def control_group() -> Optional[dist.ProcessGroup]:
    """A gloo group spanning WORLD for host object collectives (None when world is 1)."""
    global _control_pg
    if not dist.is_initialized() or dist.get_world_size() == 1:
        return None
    if _control_pg is None:
        # A group of its own even when WORLD is gloo already: the budget of every bounded wait also bounds the host
        # collectives, so a rank that never joins ends the exchange with an error instead of blocking its peers for
        # the backend's default (half an hour).  Heap bootstrap and allocation run on it too, hence the floor.
        from datetime import timedelta
        _control_pg = dist.new_group(backend="gloo",
                                     timeout=timedelta(milliseconds=max(1000, config.wait_timeout_ms())))
    return _control_pg


def reset_control_group() -> None:
    global _control_pg, _local_world_pg, _comm_stream, _heartbeat
    _control_pg = None
    _local_world_pg = None
    _comm_stream = None
    if _heartbeat is not None:
        _heartbeat.stop_background()
    _heartbeat = None


def heartbeat():
    """The job's host-side liveness channel (``ODC_HEARTBEAT_S`` > 0), created on first use; else None.

    It publishes from a background thread once a second, so a rank counts as alive while its process runs, however
    long its microbatches take; a rank that exits between steps calls ``mark_leaving`` or simply stops publishing.
    """
    global _heartbeat
    if config.heartbeat_s() <= 0 or not dist.is_initialized() or dist.get_world_size() == 1:
        return None
    if _heartbeat is None:
        from torch.distributed.distributed_c10d import _get_default_store
        from .status import Heartbeat
        _heartbeat = Heartbeat(_get_default_store(), dist.get_rank(), dist.get_world_size())
        _heartbeat.start_background(1.0)
    return _heartbeat


def check_peers_alive(missing_is_dead: bool = True) -> None:
    """Raise ``PeerFailure`` if a peer stopped publishing heartbeats (no-op unless ``ODC_HEARTBEAT_S`` is set)."""
    hb = heartbeat()
    if hb is not None:
        hb.assert_alive(config.heartbeat_s(), missing_is_dead)


def all_gather_object(obj: Any) -> List[Any]:
    pg = control_group()
    if pg is None:
        return [obj]
    out: List[Any] = [None] * dist.get_world_size()
    try:
        dist.all_gather_object(out, obj, group=pg)
    except (RuntimeError, dist.DistBackendError) as e:  # a peer never joined or went away: the group's timeout ran out
        from .status import PeerFailure
        raise PeerFailure(f"rank {rank()}: host exchange failed, a peer did not take part: {e}") from e
    return out


def broadcast_object(obj: Any, src: int = 0) -> Any:
    pg = control_group()
    if pg is None:
        return obj
    box = [obj]
    dist.broadcast_object_list(box, src=src, group=pg)
    return box[0]


def host_barrier() -> None:
    """Barrier on the control group: orders host code only, touches no CUDA stream."""
    pg = control_group()
    if pg is None:
        return
    # with heartbeats on, a rank that left is reported here instead of timing the barrier out (a peer that has not
    # published yet is still starting up: barriers run during start-up too)
    check_peers_alive(missing_is_dead=False)
    try:
        dist.barrier(group=pg)
    except (RuntimeError, dist.DistBackendError) as e:
        from .status import PeerFailure
        raise PeerFailure(f"rank {rank()}: host barrier failed, a peer did not take part: {e}") from e


def group_ranks(pg: Optional[dist.ProcessGroup]) -> List[int]:
    """Global ranks of ``pg`` in group-rank order (WORLD when ``pg`` is None)."""
    if not dist.is_initialized():
        return [0]
    if pg is None or pg is dist.group.WORLD:
        return list(range(dist.get_world_size()))
    return list(dist.get_process_group_ranks(pg))


def get_local_world_size() -> int:
    return min(config.local_world_size(world_size()), world_size())


def node_ranks(r: Optional[int] = None) -> List[int]:
    """Global ranks that share a node (one NVLink domain, one ``/dev/shm``) with rank ``r`` (default: this rank).

    Ranks of a node are contiguous: ``[r - r % L, r - r % L + L)`` with ``L`` the local world size.
    """
    ws, lws = world_size(), get_local_world_size()
    if lws <= 0 or ws % lws != 0:
        raise ValueError(f"world size {ws} is not a multiple of the local world size {lws}")
    r = rank() if r is None else r
    base = r - r % lws
    return list(range(base, base + lws))


def num_nodes() -> int:
    return world_size() // max(1, min(get_local_world_size(), world_size()))


def get_local_world_pg():
    """Per-node process groups; ranks of one node are contiguous (utils.py:180-193)."""
    global _local_world_pg
    if _local_world_pg is None and dist.is_initialized():
        lws = get_local_world_size()
        ws = dist.get_world_size()
        if ws % lws != 0:
            raise ValueError(f"world size {ws} is not a multiple of the local world size {lws}")
        mine = None
        for node in range(ws // lws):
            ranks = list(range(node * lws, (node + 1) * lws))
            pg = dist.new_group(ranks=ranks)
            if dist.get_rank() in ranks:
                mine = pg
        _local_world_pg = mine
    return _local_world_pg


def get_comm_stream():
    """The one side stream on which on-demand transfers run (utils.py:175-178)."""
    global _comm_stream
    if not torch.cuda.is_available():
        return None
    if _comm_stream is None:
        _comm_stream = torch.cuda.Stream(priority=-1)
    return _comm_stream


def job_token() -> str:
    """A string shared by all ranks of this job and unique on the host (names shm files / sockets)."""
    tok = None
    if rank() == 0:
        tok = f"{os.getpid()}_{int.from_bytes(os.urandom(4), 'little'):08x}"
    return broadcast_object(tok, src=0)
