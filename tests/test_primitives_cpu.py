"""gather / scatter_accumulate over the host-shm heap with gloo ranks (no GPU)."""
import pytest
import torch

from _mp import run_ranks


def _prim(rank, world, n, uneven):
    import odc_b200 as odc

    reg = odc.init_nvshmem("cpu", 64 << 20)
    g = odc.GatherService()
    red = odc.ReductionService(accumulation_dtype=torch.float32)
    shard = reg.allocate_symm_buffer("w", (n,), torch.float32)
    shard.copy_(torch.arange(n, dtype=torch.float32) + 1000 * rank)
    from odc_b200.runtime import control
    control.host_barrier()
    out = torch.empty(n * world, dtype=torch.bfloat16)
    g.gather_into_tensor(out, shard)
    want = torch.cat([torch.arange(n, dtype=torch.float32) + 1000 * r for r in range(world)]).to(torch.bfloat16)
    assert torch.equal(out, want)
    # scatter-accumulate: rank r contributes (r+1) rounds when uneven, else 2
    rounds = (rank + 1) if uneven else 2
    red.register("g", n, torch.bfloat16)
    for k in range(rounds):
        x = torch.full((world * n,), float(rank + 1), dtype=torch.bfloat16)
        red.scatter_accumulate("g", x)
    red.sync()
    acc = red.get_accumulation("g")
    total = sum((r + 1) * ((r + 1) if uneven else 2) for r in range(world))
    assert acc.dtype == torch.float32
    assert torch.equal(acc, torch.full((n,), float(total)))
    control.host_barrier()
    red.clear_accumulations()
    assert float(acc.abs().sum()) == 0.0
    red.stop()
    odc.finalize_distributed()
    return True


@pytest.mark.parametrize("world,uneven", [(2, False), (3, True)])
def test_primitives_host_shm(world, uneven):
    assert all(run_ranks(_prim, world, 1000, uneven))


def test_splitter(monkeypatch):
    from odc_b200 import BufferSplitter
    monkeypatch.setenv("ODC_MAX_BUFFER_SIZE", "1024")
    s = BufferSplitter()
    assert s.get_global_buffer_size((4096,)) == 1024
    assert s.get_local_buffer_size((4096,), 8) == 128
    assert s.get_local_buffer_size((100,), 8) == 128  # rounded up to 64
    assert list(s.segments(300, 8)) == [(0, 128), (128, 128), (256, 44)]
    with pytest.raises(ValueError):
        s.get_local_buffer_size((4096,), 3)
    monkeypatch.setenv("ODC_MAX_BUFFER_SIZE", "0")
    s = BufferSplitter()
    assert s.get_global_buffer_size((4096,)) == 4096
    assert s.get_local_buffer_size((4096,), 8) == 4096


def test_offset_allocator():
    from odc_b200.runtime.heap import OffsetAllocator
    a = OffsetAllocator(1 << 20)
    x, y, z = a.alloc(100), a.alloc(5000), a.alloc(1)
    assert x == 0 and y == 512 and z == 512 + 5120
    a.release(y)
    assert a.alloc(4000) == 512
    a.release(x); a.release(z)
    with pytest.raises(MemoryError):
        a.alloc(2 << 20)


def _deterministic(rank, world, trial):
    import time

    import odc_b200 as odc
    from odc_b200.runtime import control
    odc.init_nvshmem("cpu", 64 << 20)
    red = odc.ReductionService(accumulation_dtype=torch.float32)
    assert red.deterministic
    n = 4096
    red.register("g", n, torch.float32)
    g = torch.Generator().manual_seed(100 + rank)
    for k in range(2 + rank):
        time.sleep(0.001 * ((rank * 7 + trial * 3 + k) % 5))     # shuffle arrival order between trials
        red.scatter_accumulate("g", torch.randn(world * n, generator=g) * 1e3)
    red.sync()
    out = red.get_accumulation("g").clone()
    control.host_barrier()
    red.clear_accumulations()
    assert float(red.get_accumulation("g").abs().sum()) == 0.0
    red.stop()
    odc.finalize_distributed()
    return out


def test_deterministic_mode_is_bitwise_reproducible():
    runs = [run_ranks(_deterministic, 3, t, env={"ODC_DETERMINISTIC": "1"}) for t in range(2)]
    for r in range(3):
        assert torch.equal(runs[0][r], runs[1][r])
    # and it is the fixed-order sum: producers in rank order, each producer's rounds in issue order
    n = 4096
    want = torch.zeros(n)
    for p in range(3):
        g = torch.Generator().manual_seed(100 + p)
        slot = torch.zeros(n)
        for k in range(2 + p):
            slot += (torch.randn(3 * n, generator=g) * 1e3).view(3, n)[0]
        want += slot
    assert torch.equal(runs[0][0], want)


def _segments(rank, world):
    import odc_b200 as odc
    from odc_b200.runtime import control
    odc.init_nvshmem("cpu", 64 << 20)
    red = odc.ReductionService(accumulation_dtype=torch.float32)
    shapes = [(7, 5), (world * 4, 6), (3,), (world * 2 + 1, 2, 3)]  # ragged, even, shorter than the group, 3-D
    chunks, offsets, o = [], [], 0
    for s in shapes:
        rows = -(-s[0] // world)
        c = rows * int(torch.Size(s).numel() // s[0])
        chunks.append(c); offsets.append(o); o += c
    red.register("g", o, torch.bfloat16)
    gen = torch.Generator().manual_seed(7)
    all_grads = [[torch.randint(-8, 8, s, generator=gen).to(torch.bfloat16) for s in shapes] for _ in range(world)]
    for _ in range(rank + 1):  # rank r contributes r + 1 times
        assert red.scatter_accumulate_segments("g", all_grads[rank], chunks, offsets, scale=0.5)
    red.sync()
    want = torch.zeros(o)
    for r in range(world):
        for g, c, off in zip(all_grads[r], chunks, offsets):
            piece = g.reshape(-1)[rank * c:(rank + 1) * c].float()
            want[off:off + piece.numel()] += 0.5 * (r + 1) * piece
    ok = torch.equal(red.get_accumulation("g"), want)
    control.host_barrier()
    red.stop()
    odc.finalize_distributed()
    return ok


def test_scatter_accumulate_segments_matches_flattened_reduction():
    assert all(run_ranks(_segments, 3))
