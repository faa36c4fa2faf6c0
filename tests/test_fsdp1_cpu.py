"""FSDP1 with on-demand communication against stock FSDP1, on CPU ranks (gloo)."""
import pytest
import torch

from _mp import assert_mostly_close, run_pair


def _train(rank, world, mode, uneven, mp=False, fused_opt=False):
    import functools

    import torch.distributed as dist
    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
    from torch.distributed.fsdp.wrap import ModuleWrapPolicy

    import odc_b200 as odc
    from odc_b200.data import LengthSpec, make_minibatch
    from odc_b200.fsdp import fsdp1
    from odc_b200.models import DecoderLayer, DecoderLM, get_config

    seen_dtypes = set()
    if mode == "odc":
        fsdp1.patch_fsdp1(reduce_dtype=torch.float32)
        odc.init_nvshmem("cpu", 256 << 20)
        stock_scatter = odc.ReductionService.scatter_accumulate

        def recording_scatter(self, key, input, *a, **k):
            seen_dtypes.add((input.dtype, self.get_accumulation(key).dtype))
            return stock_scatter(self, key, input, *a, **k)

        odc.ReductionService.scatter_accumulate = recording_scatter
    torch.manual_seed(0)
    model = DecoderLM(get_config("tiny"))
    model.reset_parameters(seed=0)
    from torch.distributed.fsdp import MixedPrecision
    policy = MixedPrecision(param_dtype=torch.bfloat16, reduce_dtype=torch.float32) if mp else None
    model = FSDP(model, auto_wrap_policy=ModuleWrapPolicy({DecoderLayer}), device_id=torch.device("cpu"),
                 use_orig_params=False, mixed_precision=policy)
    fused_opt = fused_opt and mode == "odc"
    opt = fsdp1.FusedAdamW(model, lr=1e-3) if fused_opt else torch.optim.AdamW(model.parameters(), lr=1e-3)
    if mode == "odc":
        fsdp1.pre_minibatch_start(model)
    losses = []
    for step in range(3):
        mine = (2 + rank) if uneven else 2
        n_micro = mine if mode == "odc" else (2 + world - 1 if uneven else 2)
        total = torch.zeros(())
        for i in range(n_micro):
            real = i < mine
            mb = make_minibatch(rank, step, 1024, LengthSpec("uniform", lo=16, hi=128), mine, 128, seed=7)[i if real else 0]
            loss = model(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"], labels=mb["labels"],
                         loss_scale=mb["loss_scale"])
            if not real:
                loss = loss * 0.0
            loss.backward()
            total += loss.detach()
        if mode == "odc":
            fsdp1.pre_optimizer_step(model, materialize_grads=not fused_opt)
        if fused_opt:
            opt.clip_grad_norm_(0.5)
        elif mp:
            model.clip_grad_norm_(0.5)
        opt.step()
        opt.zero_grad()
        if mode == "odc":
            fsdp1.pre_minibatch_start(model)
        dist.all_reduce(total)
        losses.append(float(total))
    with FSDP.summon_full_params(model):
        full = {k: v.detach().clone() for k, v in model.named_parameters()}
    if mode == "odc":
        fsdp1.stop()
    return losses, full, seen_dtypes


@pytest.mark.parametrize("uneven", [False, True])
def test_fsdp1_matches_stock(uneven):
    a, b = run_pair(_train, 2, (uneven,))
    assert a[0][0] == pytest.approx(b[0][0], rel=1e-4), (a[0][0], b[0][0])
    for k in a[0][1]:
        assert_mostly_close(a[0][1][k], b[0][1][k], rtol=5e-3, atol=2e-4)


def test_fsdp1_two_emulated_nodes():
    # one rank per "node": flat-parameter gathers and gradient contributions to the peer use the inter-node path
    a, b = run_pair(_train, 2, (True,), env={"LOCAL_WORLD_SIZE": "1"})
    assert a[0][0] == pytest.approx(b[0][0], rel=1e-4), (a[0][0], b[0][0])
    for k in a[0][1]:
        assert_mostly_close(a[0][1][k], b[0][1][k], rtol=5e-3, atol=2e-4)


def test_fsdp1_mixed_precision_reduces_bf16_gradients_into_fp32_accumulators():
    a, b = run_pair(_train, 2, (True, True))
    # the unsharded gradients reach the reduction in bf16 (stock's widening pass is skipped) and land in fp32
    assert b[0][2] == {(torch.bfloat16, torch.float32)}
    assert a[0][0] == pytest.approx(b[0][0], rel=2e-2), (a[0][0], b[0][0])
    for k in a[0][1]:
        assert_mostly_close(a[0][1][k].float(), b[0][1][k].float(), rtol=2e-2, atol=3e-3, outlier_atol=1e-2)


def test_fsdp1_fused_adamw_matches_torch_adamw_with_clipping():
    """``fsdp1.FusedAdamW`` on the accumulators (mixed precision, unequal microbatch counts, clip at 0.5) against
    stock FSDP1 with ``torch.optim.AdamW`` and ``model.clip_grad_norm_``."""
    a, b = run_pair(_train, 2, (True, True, True))
    assert a[0][0] == pytest.approx(b[0][0], rel=2e-2), (a[0][0], b[0][0])
    for k in a[0][1]:
        assert_mostly_close(a[0][1][k].float(), b[0][1][k].float(), rtol=2e-2, atol=3e-3, outlier_atol=1e-2)


def _train_zero(rank, world, mode):
    """Rank 1 runs no microbatch in minibatch 1 (FSDP1)."""
    import torch.nn as nn
    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP

    import odc_b200 as odc
    from odc_b200.fsdp import fsdp1

    ragged = []
    if mode == "odc":
        fsdp1.patch_fsdp1(reduce_dtype=None)
        odc.init_nvshmem("cpu", 64 << 20)
        stock_segments = odc.ReductionService.scatter_accumulate_segments

        def recording_segments(self, key, grads, chunks, offsets, *a, **k):
            ragged.append((grads[0].numel(), chunks[0]))
            return stock_segments(self, key, grads, chunks, offsets, *a, **k)

        odc.ReductionService.scatter_accumulate_segments = recording_segments
    torch.manual_seed(0)
    net = nn.Sequential(nn.Linear(20, 32), nn.Tanh(), nn.Linear(32, 3))
    model = FSDP(net, device_id=torch.device("cpu"), use_orig_params=False)
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    if mode == "odc":
        fsdp1.pre_minibatch_start(model)
    for step in range(3):
        idle = rank == 1 and step == 1
        for i in range(2):
            if idle and mode == "odc":
                continue
            g = torch.Generator().manual_seed(100 * step + 10 * i + rank)
            x = torch.randn(5, 20, generator=g)
            y = torch.randint(0, 3, (5,), generator=g)
            loss = nn.functional.cross_entropy(model(x), y)
            (loss * (0.0 if idle else 1.0)).backward()
        if mode == "odc":
            fsdp1.pre_optimizer_step(model)
        opt.step()
        opt.zero_grad()
        if mode == "odc":
            fsdp1.pre_minibatch_start(model)
    with FSDP.summon_full_params(model):
        full = {k: v.detach().clone() for k, v in model.named_parameters()}
    if mode == "odc":
        fsdp1.stop()
        odc.ReductionService.scatter_accumulate_segments = stock_segments
    return full, ragged


def test_fsdp1_rank_with_zero_microbatches():
    a, b = run_pair(_train_zero, 2)
    for k in a[0][0]:
        torch.testing.assert_close(a[0][0][k], b[0][0][k], rtol=1e-5, atol=1e-6)
    # 771 parameters over 2 ranks: the flat gradient is reduced as ragged pieces (386 + 385), never padded with a copy
    assert b[0][1] and set(b[0][1]) == {(771, 386)}
