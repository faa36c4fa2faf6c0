"""Two emulated nodes on one machine: ranks of the other "node" are not mapped and are reached over TCP.

All listeners bind to the loopback address (the default when ``ODC_HOST_ADDR`` is not set).
"""
import pytest
import torch

from _mp import run_ranks


def _prim(rank, world, n):
    import odc_b200 as odc
    from odc_b200.runtime import control
    from odc_b200.runtime.transport import HybridTransport

    reg = odc.init_nvshmem("cpu", 64 << 20)
    lws = control.get_local_world_size()
    assert control.num_nodes() == world // lws and reg.internode is not None
    assert all(host == "127.0.0.1" for host, _ in reg.internode.addresses)
    other = (rank + lws) % world
    assert not reg.heap.is_local(other) and reg.heap.is_local(rank)
    g = odc.GatherService()
    red = odc.ReductionService(accumulation_dtype=torch.float32)
    assert isinstance(g.transport, HybridTransport)
    shard = reg.allocate_symm_buffer("w", (n,), torch.float32)
    shard.copy_(torch.arange(n, dtype=torch.float32) + 1000 * rank)
    with pytest.raises(ValueError):
        reg.heap.peer(other, reg.offset_of(shard), n, torch.float32)  # other nodes are never mapped
    peers = reg.get_peer_tensors(shard)
    assert peers[other] is None and peers[rank] is not None
    control.host_barrier()
    out = torch.empty(n * world, dtype=torch.bfloat16)
    g.gather_into_tensor(out, shard)
    want = torch.cat([torch.arange(n, dtype=torch.float32) + 1000 * r for r in range(world)]).to(torch.bfloat16)
    assert torch.equal(out, want)
    # a sub-group that lies entirely on the other node
    far = control.node_ranks(other)
    out2 = torch.empty(n * len(far), dtype=torch.float32)
    g.gather_ranks(out2, shard, far)
    assert torch.equal(out2, torch.cat([torch.arange(n, dtype=torch.float32) + 1000 * r for r in far]))
    # uneven numbers of contributions per rank, bf16 rows into fp32 accumulators
    red.register("g", n, torch.bfloat16)
    for _ in range(rank + 1):
        red.scatter_accumulate("g", torch.full((world * n,), float(rank + 1), dtype=torch.bfloat16), scale=0.5)
    red.sync()
    acc = red.get_accumulation("g")
    assert torch.equal(acc, torch.full((n,), 0.5 * sum((r + 1) ** 2 for r in range(world))))
    control.host_barrier()
    served = dict(reg.internode.served)
    sent = dict(reg.internode.sent)
    red.stop()
    odc.finalize_distributed()
    return served, sent


def test_gather_and_scatter_accumulate_across_emulated_nodes():
    world, lws, n = 4, 2, 3000
    res = run_ranks(_prim, world, n, env={"LOCAL_WORLD_SIZE": str(lws)})
    for rank, (served, sent) in enumerate(res):
        assert sent["get"] == 2 + 2          # two far ranks in the WORLD gather, two in the far sub-group
        assert sent["add"] == 2 * (rank + 1)  # every call reaches the two far owners
    assert sum(s["get"] for s, _ in res) == 4 * 4
    assert sum(s["add"] for s, _ in res) == sum(2 * (r + 1) for r in range(world))


def test_staging_cap_splits_transfers_but_counts_one_arrival_per_contribution():
    world, lws, n = 4, 2, 3000
    # 2048 elements per round over two far peers -> pieces of 1024 elements: 3 pieces per shard
    res = run_ranks(_prim, world, n, env={"LOCAL_WORLD_SIZE": str(lws), "ODC_MAX_BUFFER_SIZE": "2048"})
    for rank, (served, sent) in enumerate(res):
        assert sent["get"] == 3 * (2 + 2)
        assert sent["add"] == 3 * 2 * (rank + 1)


def _bad_request(rank, world):
    import socket

    import odc_b200 as odc
    from odc_b200.runtime import control

    reg = odc.init_nvshmem("cpu", 1 << 20)
    ok = True
    if rank == 0:
        try:  # a range outside the owner's region is refused by the server, which keeps serving
            reg.internode.get_many([1], (1 << 20) - 16, 1024, torch.float32)
            ok = False
        except RuntimeError as e:
            ok = "IndexError" in str(e)
        buf = reg.internode.get_many([1], 0, 4, torch.int32)[0]
        ok = ok and buf.numel() == 4
        # a connection that cannot answer the challenge with the job's secret is closed unserved
        host, port = reg.internode.addresses[1]
        with socket.create_connection((host, port), timeout=10) as c:
            c.settimeout(10)
            c.recv(16)
            c.sendall(b"x" * 32)
            ok = ok and c.recv(64) == b""  # closed without an answer
    control.host_barrier()
    if rank == 1:
        ok = ok and reg.internode.rejected == 1 and reg.internode.served["get"] == 1
    odc.finalize_distributed()
    return ok


def test_server_rejects_out_of_range_requests_and_strangers():
    assert all(run_ranks(_bad_request, 2, env={"LOCAL_WORLD_SIZE": "1"}))


def test_wildcard_bind_address_is_refused(monkeypatch):
    from odc_b200.runtime import internode
    monkeypatch.delenv("ODC_HOST_ADDR", raising=False)
    assert internode._bind_address() == "127.0.0.1"
    monkeypatch.setenv("ODC_HOST_ADDR", "0.0.0.0")
    with pytest.raises(ValueError):
        internode._bind_address()


def _linear(rank, world):
    import odc_b200 as odc
    from odc_b200 import parallel
    from odc_b200.runtime import control
    odc.init_nvshmem("cpu", 64 << 20)
    lin = parallel.OdcLinear(32, 50, seed=3)
    torch.manual_seed(100 + rank)
    xs = [torch.randn(5 + rank, 32, requires_grad=True) for _ in range(1 + rank)]
    parallel.start_minibatch()
    ys = []
    for x in xs:
        y = lin(x)
        y.pow(2).sum().backward()
        ys.append(y.detach())
    shard = lin.weight.master.clone()
    parallel.finish_minibatch(lr=0.0)
    out = dict(xs=[x.detach() for x in xs], dxs=[x.grad for x in xs], ys=ys, grad=lin.weight.grad().clone(), shard=shard)
    control.host_barrier()
    parallel.reset()
    odc.finalize_distributed()
    return out


def test_sharded_linear_layer_across_emulated_nodes():
    world = 2
    res = run_ranks(_linear, world, env={"LOCAL_WORLD_SIZE": "1"})
    W = torch.cat([r["shard"] for r in res])[:50].bfloat16().float()
    dW = torch.zeros(50, 32)
    for r in res:
        for x, y, dx in zip(r["xs"], r["ys"], r["dxs"]):
            want = x @ W.t()
            torch.testing.assert_close(y, want, rtol=1e-4, atol=1e-4)
            torch.testing.assert_close(dx, (2 * want) @ W, rtol=1e-4, atol=1e-4)
            dW += (2 * want).t() @ x
    torch.testing.assert_close(torch.cat([r["grad"] for r in res])[:50], dW / world, rtol=1e-4, atol=1e-4)
