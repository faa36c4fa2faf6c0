"""Failure detection without touching a GPU: failures are made on the host, between CPU ranks."""
import random

import pytest
import torch

from _mp import run_ranks


def _dropped_contribution(rank, world):
    """Rank 1 announces a contribution that never arrives: owners' bounded wait must report, not hang."""
    import odc_b200 as odc
    from odc_b200.runtime import control
    from odc_b200.runtime.status import OdcTimeoutError
    reg = odc.init_nvshmem("cpu", 32 << 20)
    red = odc.ReductionService(accumulation_dtype=torch.float32)
    red.register("g", 64, torch.float32)
    red.scatter_accumulate("g", torch.ones(world * 64))
    if rank == 1:
        red.note_dispatch(list(range(world)))  # the message itself is "dropped": counted but never sent
    control.host_barrier()   # both ranks enter sync together, so the short wait below measures the missing arrival only
    timed_out = False
    try:
        red.sync()
    except OdcTimeoutError as e:
        timed_out = True
        assert "arrived within" in str(e)
    # the runtime is still usable afterwards: a gather works
    shard = reg.allocate_symm_buffer("w", (16,), torch.float32)
    shard.fill_(float(rank))
    control.host_barrier()
    out = torch.empty(world * 16)
    odc.GatherService().gather_into_tensor(out, shard)
    assert out.view(world, 16)[:, 0].tolist() == [float(r) for r in range(world)]
    control.host_barrier()
    odc.finalize_distributed()
    return timed_out


def test_wait_reports_a_missing_contribution():
    res = run_ranks(_dropped_contribution, 2, env={"ODC_WAIT_TIMEOUT_MS": "1500"})
    assert all(res)  # every owner was told to expect one more arrival than it received


def _never_posts(rank, world):
    """One-sided count exchange: rank 1 never reaches `sync`, so its posting is missing on every owner."""
    import odc_b200 as odc
    from odc_b200.runtime.status import OdcTimeoutError
    odc.init_nvshmem("cpu", 32 << 20)
    red = odc.ReductionService(accumulation_dtype=torch.float32)
    red.register("g", 64, torch.float32)
    red.scatter_accumulate("g", torch.ones(world * 64))
    if rank == 1:
        return "absent"          # between steps, nothing in flight; it simply does not take part
    with pytest.raises(OdcTimeoutError, match="did not post"):
        red.sync()
    return "reported"


def test_sync_reports_a_producer_that_never_posts():
    assert run_ranks(_never_posts, 2, env={"ODC_WAIT_TIMEOUT_MS": "400"}) == ["reported", "absent"]


def _never_joins_host_exchange(rank, world):
    """`sync` with a payload uses one host exchange; its group carries the wait budget, so an absent rank is an error."""
    import time

    import odc_b200 as odc
    from odc_b200.runtime.status import PeerFailure
    odc.init_nvshmem("cpu", 32 << 20)
    red = odc.ReductionService(accumulation_dtype=torch.float32)
    red.register("g", 64, torch.float32)
    if rank == 1:
        time.sleep(3.0)          # stays alive (so the store stays up) but never calls sync
        return "absent"
    t0 = time.monotonic()
    with pytest.raises(PeerFailure, match="did not take part"):
        red.sync(payload={"anything": 1})
    assert time.monotonic() - t0 < 30
    return "reported"


def test_host_exchange_is_bounded_by_the_wait_budget():
    assert run_ranks(_never_joins_host_exchange, 2, env={"ODC_WAIT_TIMEOUT_MS": "1000"}) == ["reported", "absent"]


def _left_between_steps(rank, world):
    """With ODC_HEARTBEAT_S set, `sync` learns on the host that a peer left, before it waits for anything."""
    import time

    import odc_b200 as odc
    from odc_b200.runtime import control
    from odc_b200.runtime.status import PeerFailure
    odc.init_nvshmem("cpu", 32 << 20)
    red = odc.ReductionService(accumulation_dtype=torch.float32)
    red.register("g", 64, torch.float32)
    red.scatter_accumulate("g", torch.ones(world * 64))
    red.sync()                   # a normal minibatch first: everyone is alive
    control.host_barrier()
    if rank == 1:
        control.heartbeat().mark_leaving()
        time.sleep(3.0)
        return "left"
    time.sleep(1.0)
    t0 = time.monotonic()
    with pytest.raises(PeerFailure, match="stopped publishing"):
        red.sync()
    assert time.monotonic() - t0 < 5.0   # none of the 20 s wait budget was spent
    return "detected"


def test_sync_checks_heartbeats_first():
    res = run_ranks(_left_between_steps, 2, env={"ODC_HEARTBEAT_S": "30", "ODC_WAIT_TIMEOUT_MS": "20000"})
    assert res == ["detected", "left"]


def _heartbeat(rank, world):
    import time

    import torch.distributed as dist

    from odc_b200.runtime.status import Heartbeat, PeerFailure
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world)
    hb.beat(0)
    dist.barrier()
    assert hb.dead_peers(max_age_s=30.0) == []
    dist.barrier()  # everyone has looked before anyone leaves
    if rank == 1:
        hb.mark_leaving()  # leaves between steps, nothing in flight
        dist.barrier()
        return "left"
    dist.barrier()
    dead = hb.dead_peers(max_age_s=30.0)
    assert dead == [1], dead
    with pytest.raises(PeerFailure):
        hb.assert_alive(30.0)
    # a peer that simply stops publishing is caught by age
    time.sleep(0.3)
    hb.beat(1)
    stale = hb.dead_peers(max_age_s=0.1)
    assert 1 in stale
    return "detected"


def test_heartbeat_detects_a_rank_that_left():
    assert run_ranks(_heartbeat, 2) == ["detected", "left"]


def _raises(rank, world):
    if rank == 1:
        raise ValueError("injected host failure on rank 1")
    return True


def test_a_raising_rank_is_reported():
    with pytest.raises(RuntimeError, match="injected host failure"):
        run_ranks(_raises, 2, timeout=60)


def test_heap_views_are_bounds_checked():
    from odc_b200.runtime.heap import OffsetAllocator
    from odc_b200.runtime.status import OdcBoundsError, check_status_word
    a = OffsetAllocator(4096)
    a.alloc(4096)
    with pytest.raises(MemoryError):
        a.alloc(1)
    with pytest.raises(OdcBoundsError):
        check_status_word(2, 3, 0)
    check_status_word(0)


# ------------------------------------------------------------------------------------------
# host model of the arrival protocol: reductions, then fence, then one release on the counter
# ------------------------------------------------------------------------------------------
def _simulate(n_producers, n_chunks, signal_first, seed):
    """Returns True if the owner, once it has seen all arrivals, always reads the complete sum."""
    rng = random.Random(seed)
    progs = []
    for p in range(n_producers):
        ops = [("add", p, c) for c in range(n_chunks)]
        ops = [("signal", p, None)] + ops if signal_first else ops + [("signal", p, None)]
        progs.append(ops)
    pcs = [0] * n_producers
    acc = [0] * n_chunks
    counter = 0
    while any(pc < len(pr) for pc, pr in zip(pcs, progs)):
        p = rng.choice([i for i in range(n_producers) if pcs[i] < len(progs[i])])
        op, _, c = progs[p][pcs[p]]
        pcs[p] += 1
        if op == "add":
            acc[c] += p + 1
        else:
            counter += 1
        if counter == n_producers:  # the owner's wait is satisfied here: it may read now
            if acc != [sum(range(1, n_producers + 1))] * n_chunks:
                return False
    return True


def test_arrival_protocol_model():
    assert all(_simulate(4, 5, signal_first=False, seed=s) for s in range(200))
    # negative control: signalling before the data is out is caught by some interleaving
    assert not all(_simulate(4, 5, signal_first=True, seed=s) for s in range(200))


def _far_peer_gone(rank, world):
    """Inter-node path: an owner whose server is gone, or that never answers, gives an error within the wait budget."""
    import socket
    import time

    import odc_b200 as odc
    from odc_b200.runtime import control
    from odc_b200.runtime.status import OdcTimeoutError

    reg = odc.init_nvshmem("cpu", 1 << 20)
    ep = reg.internode
    out = {}
    if rank == 1:
        ep.close()           # this rank "left" between steps: nobody listens on its port any more
    control.host_barrier()
    if rank == 0:
        t0 = time.monotonic()
        try:
            ep.get_many([1], 0, 4, torch.int32)
            out["refused"] = False
        except OSError:
            out["refused"] = True
        # an owner that accepts the connection but never speaks: the challenge does not arrive in time
        silent = socket.socket()
        silent.bind(("127.0.0.1", 0))
        silent.listen(1)
        ep.addresses[1] = silent.getsockname()
        try:
            ep.get_many([1], 0, 4, torch.int32)
            out["timed_out"] = False
        except OdcTimeoutError:
            out["timed_out"] = True
        silent.close()
        out["seconds"] = time.monotonic() - t0
    control.host_barrier()
    odc.finalize_distributed()
    return out


def test_inter_node_owner_that_left_or_stalls_is_reported():
    res = run_ranks(_far_peer_gone, 2, env={"LOCAL_WORLD_SIZE": "1", "ODC_WAIT_TIMEOUT_MS": "500"})
    assert res[0]["refused"] and res[0]["timed_out"] and res[0]["seconds"] < 10
