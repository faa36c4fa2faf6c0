"""Packing / load balancing and the synthetic workloads (pure CPU)."""
import numpy as np
import pytest
import torch

from odc_b200.data import (BatchedDataset, LengthSpec, balanced_partitions, bin_pack_decreasing, get_cost_fn,
                           get_packing_function, greedy_partition, imbalance_report, karmarkar_karp, make_minibatch,
                           pack_microbatch, rearrange_micro_batches, sample_lengths)


def _lengths(kind, n, seed=0):
    spec = {"lognormal": LengthSpec("lognormal", lo=16, median=512, sigma=1.0, cap=8192),
            "longtail": LengthSpec("longtail"), "uniform": LengthSpec("uniform", lo=16, hi=128)}[kind]
    return sample_lengths(spec, n, np.random.default_rng(seed))


def test_length_distributions_respect_their_bounds():
    ln = _lengths("lognormal", 4000)
    assert 16 <= min(ln) and max(ln) <= 8192 and 350 < float(np.median(ln)) < 700
    lt = _lengths("longtail", 4000)
    long_frac = sum(x >= 8192 for x in lt) / len(lt)
    assert 0.2 < long_frac < 0.3 and all((256 <= x <= 2048) or (8192 <= x <= 32768) for x in lt)


@pytest.mark.parametrize("k", [2, 4, 8])
@pytest.mark.parametrize("equal", [False, True])
def test_karmarkar_karp_is_a_partition_and_balances(k, equal):
    L = _lengths("longtail", 64, seed=k)
    parts = karmarkar_karp([float(x) for x in L], k, equal_size=equal)
    assert sorted(i for p in parts for i in p) == list(range(64))
    if equal:
        assert {len(p) for p in parts} == {64 // k}
    loads = [sum(L[i] for i in p) for p in parts]
    greedy = [sum(L[i] for i in p) for p in greedy_partition([float(x) for x in L], k, equal_size=equal)]
    assert sorted(i for p in greedy_partition([float(x) for x in L], k, equal_size=equal) for i in p) == list(range(64))
    assert max(loads) - min(loads) <= max(L)             # differencing keeps the spread below the largest item
    assert len(greedy) == k
    refined = balanced_partitions(L, k, equal_size=equal)
    rl = [sum(L[i] for i in p) for p in refined]
    assert max(rl) - min(rl) <= max(loads) - min(loads)


def test_bin_packing_respects_capacity_and_covers_everything():
    L = _lengths("lognormal", 200, seed=3)
    for best in (True, False):
        bins = bin_pack_decreasing(16384, L, best_fit=best)
        assert sorted(i for b in bins for i in b) == list(range(200))
        assert all(sum(L[i] for i in b) <= 16384 for b in bins)
        assert len(bins) <= int(np.ceil(sum(L) / 16384)) + 3
    with pytest.raises(ValueError):
        bin_pack_decreasing(100, [50, 101])


def test_rearrange_micro_batches_budget_and_order():
    L = _lengths("lognormal", 40, seed=5)
    parts = rearrange_micro_batches(L, 8192, cost_fn=get_cost_fn("fit"))
    assert sorted(i for p in parts for i in p) == list(range(40))
    assert all(sum(L[i] for i in p) <= 8192 for p in parts)
    costs = [sum(get_cost_fn("fit")([L[i] for i in p])) for p in parts]
    assert costs == sorted(costs, reverse=True)          # heaviest microbatch first


def test_strategies_cover_the_batch_once_across_ranks():
    L = _lengths("lognormal", 64, seed=7)
    for method in ("None", "LocalSort", "DebugUneven", "DynamicSameMicro", "DynamicDiffMicro"):
        fn = get_packing_function(method, max_token_len=16384, cost_fn=get_cost_fn("linear"))
        per_rank = [fn(L, r, 4) for r in range(4)]
        assert sorted(i for mbs in per_rank for mb in mbs for i in mb) == list(range(64)), method
        if method in ("DynamicSameMicro", "DynamicDiffMicro"):
            assert all(sum(L[i] for i in mb) <= 16384 for mbs in per_rank for mb in mbs)
    uneven = [len(get_packing_function("DebugUneven")(L, r, 4)) for r in range(4)]
    assert len(set(uneven)) > 1                           # ranks really get different microbatch counts
    with pytest.raises(ValueError):
        get_packing_function("DynamicDiffMicro", odc_enabled=False)


def test_imbalance_report_shows_the_bubble_lockstep_pays():
    L = _lengths("longtail", 64, seed=11)
    rep = imbalance_report(L, 8, 32768, get_cost_fn("fit"))
    assert rep["ondemand_cost"] <= rep["lockstep_cost"] + 1e-9
    assert rep["ondemand_bubble"] < 0.15 and rep["lockstep_bubble"] >= rep["ondemand_bubble"]


def test_pack_microbatch_layout():
    seqs = [torch.arange(5), torch.arange(10, 13)]
    mb = pack_microbatch(seqs, minibatch_num_seqs=4)
    assert mb["cu_seqlens"].tolist() == [0, 5, 8] and mb["position_ids"].tolist() == [0, 1, 2, 3, 4, 0, 1, 2]
    assert mb["labels"].tolist() == [1, 2, 3, 4, -100, 11, 12, -100]          # next token, none across a boundary
    assert mb["loss_scale"][0].item() == pytest.approx(1 / 5 / 4) and mb["loss_scale"][4].item() == 0.0
    assert mb["max_seqlen"] == 5 and mb["num_tokens"] == 8


def test_make_minibatch_is_seeded_per_rank_and_step():
    a = make_minibatch(0, 0, 1000, LengthSpec("uniform", lo=16, hi=128), 3, 512, seed=1)
    b = make_minibatch(0, 0, 1000, LengthSpec("uniform", lo=16, hi=128), 3, 512, seed=1)
    c = make_minibatch(1, 0, 1000, LengthSpec("uniform", lo=16, hi=128), 3, 512, seed=1)
    assert all(torch.equal(x["input_ids"], y["input_ids"]) for x, y in zip(a, b))
    assert any(x["num_tokens"] != y["num_tokens"] or not torch.equal(x["input_ids"], y["input_ids"]) for x, y in zip(a, c))
    assert all(mb["num_tokens"] <= 512 for mb in a)


def test_batched_dataset_limits_and_pads():
    rng = np.random.default_rng(0)
    seqs = [torch.from_numpy(rng.integers(0, 100, size=n)) for n in [10, 3000, 20, 30, 40, 50, 60, 70]]
    ds = BatchedDataset(seqs, batch_size=4, rank=0, world_size=2, packing_method="DynamicDiffMicro", max_token_len=4096,
                        limit_token_len=100)
    assert len(ds) == 1
    mbs = ds[0]
    assert sum(mb["num_seqs"] for mb in mbs) >= 3 and all(mb["num_tokens"] <= 4096 for mb in mbs)
    assert "rank 0" in ds.last_debug


def test_report_cli_shows_the_long_tail_bubble(capsys):
    import json

    from odc_b200.data.packing import report_main
    report_main(["--world", "8", "--sequences", "64", "--dist", "longtail", "--max-token-len", "32768", "--cap", "32768",
                 "--minibatches", "5"])
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["lockstep_idle_share_mean"] > 3 * out["ondemand_idle_share_mean"]
    assert 0.0 <= out["ondemand_idle_share_mean"] < 0.1
