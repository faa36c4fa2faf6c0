"""Property tests (hypothesis) of the pure host-side pieces the symmetric heap and the primitives rely on."""
import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

# the same examples on every run: a suite that is run with -x must not depend on the draw
settings.register_profile("fixed", derandomize=True, deadline=None, database=None)
settings.load_profile("fixed")


@settings(max_examples=150, deadline=None)
@given(st.lists(st.one_of(st.tuples(st.just("a"), st.integers(1, 40000)), st.tuples(st.just("f"), st.integers(0, 64))),
                min_size=1, max_size=60))
def test_offset_allocator_never_overlaps_and_is_a_function_of_the_call_sequence(ops):
    """Ranks run the same allocation sequence and must get the same offsets: that is what makes the heap symmetric."""
    from odc_b200.runtime.heap import ALIGN, OffsetAllocator
    a, b = OffsetAllocator(1 << 20), OffsetAllocator(1 << 20)
    live = []
    for kind, x in ops:
        if kind == "a":
            try:
                off = a.alloc(x)
            except MemoryError:
                with pytest.raises(MemoryError):
                    b.alloc(x)
                continue
            assert b.alloc(x) == off and off % ALIGN == 0
            live.append((off, x))
        elif live:
            off, _ = live.pop(x % len(live))
            a.release(off)
            b.release(off)
        spans = sorted((o, o + max(n, 1)) for o, n in live)
        assert all(s1[1] <= s2[0] for s1, s2 in zip(spans, spans[1:]))       # no two live buffers overlap
        assert all(e <= 1 << 20 for _, e in spans)
        assert a.bytes_in_use + sum(s for _, s in a.free) == 1 << 20         # nothing is lost
        assert all(f1[0] + f1[1] < f2[0] for f1, f2 in zip(a.free, a.free[1:]))  # free list sorted and coalesced
    for off, _ in live:
        a.release(off)
    assert a.free == [(0, 1 << 20)] and a.high_water == 0


@settings(max_examples=200, deadline=None)
@given(st.integers(0, 100000), st.integers(1, 16), st.integers(-1, 4096))
def test_splitter_segments_tile_the_shard(numel, world, cap_units):
    from odc_b200 import BufferSplitter
    cap = cap_units * world  # the cap must be a multiple of the group size
    s = BufferSplitter(cap)
    segs = list(s.segments(numel, world))
    assert sum(n for _, n in segs) == numel
    pos = 0
    for start, n in segs:
        assert start == pos and n > 0
        pos += n
    if cap > 0 and numel > 0:
        assert max(n for _, n in segs) <= max(64, (cap // world + 63) // 64 * 64)


@settings(max_examples=100, deadline=None)
@given(st.lists(st.integers(1, 5000), min_size=1, max_size=80), st.integers(1, 8), st.booleans())
def test_partitions_and_bins_cover_every_sequence_once(lengths, k, equal):
    from odc_b200.data.packing import bin_pack_decreasing, greedy_partition, karmarkar_karp, refine_by_swaps
    if equal and len(lengths) % k != 0:
        lengths = lengths + [1] * (k - len(lengths) % k)
    costs = [float(x) for x in lengths]
    for parts in (karmarkar_karp(costs, k, equal), greedy_partition(costs, k, equal)):
        assert len(parts) == k
        assert sorted(i for p in parts for i in p) == list(range(len(costs)))
        if equal:
            assert len({len(p) for p in parts}) == 1
        refined = refine_by_swaps(costs, [list(p) for p in parts])
        assert sorted(i for p in refined for i in p) == list(range(len(costs)))
        spread = lambda ps: max(sum(costs[i] for i in p) for p in ps) - min(sum(costs[i] for i in p) for p in ps)
        assert spread(refined) <= spread(parts) + 1e-9       # swapping never makes the balance worse
    cap = max(lengths) + 100
    for best_fit in (True, False):
        bins = bin_pack_decreasing(cap, lengths, best_fit)
        assert sorted(i for b in bins for i in b) == list(range(len(lengths)))
        assert all(sum(lengths[i] for i in b) <= cap for b in bins)


@settings(max_examples=60, deadline=None)
@given(st.lists(st.integers(1, 3000), min_size=1, max_size=60), st.integers(1, 4))
def test_every_strategy_hands_each_sequence_to_exactly_one_rank(lengths, world):
    from odc_b200.data.packing import get_packing_function
    for method in ("None", "LocalSort", "DebugUneven", "DynamicSameMicro", "DynamicDiffMicro"):
        batch = list(lengths)
        if method == "DynamicSameMicro" and len(batch) % world != 0:
            batch += [1] * (world - len(batch) % world)  # equal-sized minibatches need a divisible batch
        fn = get_packing_function(method, max_token_len=4096)
        seen = []
        for rank in range(world):
            for mb in fn(batch, rank, world):
                if method.startswith("Dynamic"):
                    assert sum(batch[i] for i in mb) <= 4096
                seen += list(mb)
        assert sorted(seen) == list(range(len(batch))), method
