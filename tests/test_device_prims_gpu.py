"""One test per device-side communication primitive (loop-back on one GPU through the symmetric heap)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def heap():
    import odc_b200 as odc
    torch.cuda.set_device(0)
    reg = odc.init_nvshmem(torch.device("cuda", 0), 1 << 30)
    yield reg
    odc.finalize_distributed()


@pytest.fixture(scope="module")
def ext():
    from odc_b200 import _ext
    return _ext.load()


@pytest.mark.parametrize("n", [4, 1024, 4096 * 7 + 4])
def test_put_block_full_half_single(ext, heap, n):
    dst = heap.allocate_symm_buffer(f"put{n}", (2 * n,), torch.float32)
    dst.fill_(-1.0)
    src = torch.arange(n, device="cuda", dtype=torch.float32)
    peer_addr = heap.heap.peer_ptr(heap.heap.rank, heap.offset_of(dst))   # "remote" address of dst (loop-back)
    ext.put_block(peer_addr, src)
    torch.cuda.synchronize()
    assert torch.equal(dst[:n], src)
    assert float((dst[n:] + 1.0).abs().sum()) == 0.0            # the tail past the message is untouched
    heap.deallocate_symm_buffer(f"put{n}")


@pytest.mark.parametrize("n", [4, 1024, 4096 * 7 + 4])
def test_get_block(ext, heap, n):
    src = heap.allocate_symm_buffer(f"get{n}", (n,), torch.float32)
    src.copy_(torch.arange(n, device="cuda", dtype=torch.float32) * 2)
    out = torch.full((n + 8,), -1.0, device="cuda")
    ext.get_block(out[:n], heap.heap.peer_ptr(0, heap.offset_of(src)))
    torch.cuda.synchronize()
    assert torch.equal(out[:n], src) and float((out[n:] + 1.0).abs().sum()) == 0.0
    heap.deallocate_symm_buffer(f"get{n}")


def test_scalar_put_and_get(ext, heap):
    word = heap.allocate_symm_buffer("word", (4,), torch.int32)
    word.zero_()
    back = torch.zeros(1, dtype=torch.int32, device="cuda")
    ext.scalar_put_get(heap.heap.peer_ptr(0, heap.offset_of(word)), 42, back)
    torch.cuda.synchronize()
    assert int(word[0]) == 42 and int(back[0]) == 42
    heap.deallocate_symm_buffer("word")


def test_atomic_cas_and_swap(ext, heap):
    ctas = 10
    word = heap.allocate_symm_buffer("atom", (4,), torch.int32)
    word[0] = 5
    word[1] = 5
    cas = torch.zeros(ctas, dtype=torch.int32, device="cuda")
    swp = torch.zeros(ctas, dtype=torch.int32, device="cuda")
    ext.atomic_test(word, cas, swp, 5, 100, 100)
    torch.cuda.synchronize()
    assert int(word[0]) == 100 and int(word[1]) == 100
    assert sorted(cas.tolist()) == [5] + [100] * (ctas - 1)      # exactly one CAS saw the old value
    assert sorted(swp.tolist()) == [5] + [100] * (ctas - 1)      # exactly one swap displaced the old value
    heap.deallocate_symm_buffer("atom")


def test_bounded_grid_barrier(ext):
    ctas = 64
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    slots = torch.zeros(ctas, dtype=torch.int32, device="cuda")
    out = torch.zeros(ctas, dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ext.grid_barrier_test(counter, slots, out, 2000, status)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    assert out.tolist() == [1000 + (i + 1) % ctas for i in range(ctas)]
    # a barrier that expects more arrivals than there are CTAs gives up after its budget and reports
    counter.zero_()
    out2 = torch.zeros(ctas - 1, dtype=torch.int32, device="cuda")
    # (ctas - 1 CTAs arrive, but the counter already holds nothing: emulate a missing CTA by a pre-set deficit)
    counter.fill_(-1)
    ext.grid_barrier_test(counter, slots, out2, 50, status)
    torch.cuda.synchronize()
    assert int(status[0]) == 1 and out2.tolist() == [-1] * (ctas - 1)
