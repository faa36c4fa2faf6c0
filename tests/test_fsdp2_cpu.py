"""FSDP2 with on-demand communication against stock FSDP2, on CPU ranks (gloo)."""
import pytest
import torch

from _mp import assert_mostly_close, run_pair


def _make_batches(rank, step, n_micro, vocab=1024):
    from odc_b200.data import LengthSpec, make_minibatch
    return make_minibatch(rank, step, vocab, LengthSpec("uniform", lo=16, hi=128), n_micro, 128, seed=7)


def _train(rank, world, mode, steps, uneven, mesh_shape, hpz, mp):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    import odc_b200 as odc
    from odc_b200.fsdp import fsdp2
    from odc_b200.models import DecoderLM, get_config

    torch.manual_seed(0)
    model = DecoderLM(get_config("tiny"))
    model.reset_parameters(seed=0)
    if mode == "odc":
        odc.init_nvshmem("cpu", 256 << 20)
        fsdp2.patch_fsdp2(enable_hpz=bool(hpz))
    mesh = init_device_mesh("cpu", mesh_shape, mesh_dim_names=("rep", "shard")[-len(mesh_shape):])
    kw = dict(mesh=mesh)
    if mp:
        kw["mp_policy"] = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    raf = hpz if hpz else True
    for layer in model.layers:
        fully_shard(layer, reshard_after_forward=raf, **kw)
    fully_shard(model, reshard_after_forward=raf, **kw)
    if mode == "odc":
        for m in list(model.layers) + [model]:
            fsdp2.patch_lazy_init(m)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    losses = []
    for step in range(steps):
        if mode == "odc":
            fsdp2.pre_minibatch_start(model)
        n_micro = (2 + rank) if uneven else 2
        if uneven and mode == "stock":
            n_micro = 2 + world - 1  # lock-step FSDP must run the same count: pad with empty work below
        total = torch.zeros(())
        for i in range(n_micro):
            real = i < ((2 + rank) if uneven else 2)
            mb = _make_batches(rank, step, (2 + rank) if uneven else 2)[i if real else 0]
            loss = model(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"],
                         labels=mb["labels"], loss_scale=mb["loss_scale"])
            if not real:
                loss = loss * 0.0
            loss.backward()
            total += loss.detach()
        if mode == "odc":
            fsdp2.pre_optimizer_step(model)
        opt.step()
        opt.zero_grad()
        dist.all_reduce(total)
        losses.append(float(total))
    full = {k: v.full_tensor().clone() for k, v in model.state_dict().items()}
    breakdown = fsdp2.get_symm_buffer_memory_breakdown() if mode == "odc" else None
    if mode == "odc":
        fsdp2.stop()
    return losses, full, breakdown


def _compare(world, **kw):
    a, b = run_pair(_train, world, (4, kw.get("uneven", False), kw.get("mesh", (world,)), 0, kw.get("mp", False)),
                    (4, kw.get("uneven", False), kw.get("mesh", (world,)), kw.get("hpz", 0), kw.get("mp", False)),
                    env=kw.get("env"))
    la, lb = a[0][0], b[0][0]
    tol = 2e-2 if kw.get("mp") else 1e-4
    assert la == pytest.approx(lb, rel=tol), (la, lb)
    assert all(x == x for x in lb)
    for k in a[0][1]:
        assert_mostly_close(a[0][1][k], b[0][1][k], rtol=max(tol, 5e-3), atol=max(tol * 0.1, 2e-4))
    return b


def test_fsdp2_loss_parity_world2():
    b = _compare(2)
    assert b[0][2]["fsdp_params"] > 0 and b[0][2]["accumulation"] > 0


def test_fsdp2_uneven_microbatches():
    _compare(2, uneven=True)


def test_fsdp2_mixed_precision():
    b = _compare(2, mp=True)
    assert b[0][2]["lowp_replica"] > 0


def test_fsdp2_hsdp():
    _compare(4, mesh=(2, 2))


def test_fsdp2_hpz():
    b = _compare(4, hpz=2)
    assert b[0][2]["hpz_buffer"] > 0


def test_fsdp2_two_emulated_nodes_uneven_mixed_precision():
    # one rank per "node": every gather and every gradient contribution to the peer crosses the TCP path
    _compare(2, uneven=True, mp=True, env={"LOCAL_WORLD_SIZE": "1"})


def test_fsdp2_hpz_across_emulated_nodes():
    # two nodes of two ranks: the per-minibatch refresh pulls from both nodes, later unshards stay on the node
    b = _compare(4, hpz=2, env={"LOCAL_WORLD_SIZE": "2"})
    assert b[0][2]["hpz_buffer"] > 0


def _train_fused(rank, world, mode):
    """HSDP (2 x 2) + secondary partition of 2 + activation checkpointing; on-demand side uses FusedAdamW."""
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import odc_b200 as odc
    from odc_b200.fsdp import fsdp2
    from odc_b200.models import DecoderLM, get_config

    model = DecoderLM(get_config("tiny", activation_checkpointing=True))
    model.reset_parameters(seed=0)
    if mode == "odc":
        odc.init_nvshmem("cpu", 256 << 20)
        fsdp2.patch_fsdp2(enable_hpz=True)
    mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("rep", "shard"))
    raf = 2 if mode == "odc" else True
    for layer in model.layers:
        fully_shard(layer, mesh=mesh, reshard_after_forward=raf)
    fully_shard(model, mesh=mesh, reshard_after_forward=raf)
    if mode == "odc":
        for m in list(model.layers) + [model]:
            fsdp2.patch_lazy_init(m)
        opt = fsdp2.FusedAdamW(model, lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    else:
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    norms = []
    for step in range(3):
        if mode == "odc":
            fsdp2.pre_minibatch_start(model)
        for i in range(2):
            mb = _make_batches(rank, step, 2)[i]
            loss = model(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"],
                         labels=mb["labels"], loss_scale=mb["loss_scale"])
            loss.backward()
        if mode == "odc":
            fsdp2.pre_optimizer_step(model, materialize_grads=False)
            norms.append(float(opt.clip_grad_norm_(1e9)))
        else:
            norms.append(float(torch.nn.utils.clip_grad_norm_(model.parameters(), 1e9).full_tensor()))
        opt.step()
        opt.zero_grad()
    full = {k: v.full_tensor().clone() for k, v in model.state_dict().items()}
    if mode == "odc":
        fsdp2.stop()
    return norms, full


def test_fsdp2_hsdp_hpz_checkpointing_fused_adamw():
    a, b = run_pair(_train_fused, 4)
    assert a[0][0] == pytest.approx(b[0][0], rel=1e-3), (a[0][0], b[0][0])
    for k in a[0][1]:
        assert_mostly_close(a[0][1][k], b[0][1][k], rtol=5e-3, atol=2e-4)


def _train_partial(rank, world, mode):
    """Frozen parameters, a branch that some microbatches skip, and a unit that one rank does not run at all.

    Lock-step FSDP needs every rank to produce the same set of gradients in every backward, so the stock run
    executes the skipped parts with weight zero; the on-demand run really skips them.  The mathematics is the same.
    """
    import torch.distributed as dist
    import torch.nn as nn
    from torch.distributed.fsdp import fully_shard

    import odc_b200 as odc
    from odc_b200.fsdp import fsdp2

    skip_for_real = mode == "odc"

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Linear(24, 24)
            self.b = nn.Linear(24, 24)               # skipped by some microbatches: no gradient in that backward
            self.c = nn.Linear(24, 24, bias=False)   # frozen
            self.side = nn.Sequential(nn.Linear(24, 24), nn.Tanh())  # its own unit; rank 1 skips it in step 1
            self.head = nn.Linear(24, 5)

        def forward(self, x, use_b, use_side):
            h = torch.tanh(self.a(x))
            if use_b or not skip_for_real:
                h = h + self.b(h) * (1.0 if use_b else 0.0)
            h = self.c(h)
            if use_side or not skip_for_real:
                h = h + self.side(h) * (1.0 if use_side else 0.0)
            return self.head(h)

    torch.manual_seed(0)
    model = Net()
    model.c.weight.requires_grad_(False)
    if mode == "odc":
        odc.init_nvshmem("cpu", 64 << 20)
        fsdp2.patch_fsdp2()
    fully_shard(model.side)
    fully_shard(model)
    if mode == "odc":
        for m in (model.side, model):
            fsdp2.patch_lazy_init(m)
    opt = torch.optim.SGD([p for p in model.parameters() if p.requires_grad], lr=0.05)
    losses = []
    for step in range(3):
        if mode == "odc":
            fsdp2.pre_minibatch_start(model)
        total = torch.zeros(())
        for i in range(3):
            g = torch.Generator().manual_seed(1000 * step + 10 * i + rank)
            x = torch.randn(6, 24, generator=g)
            y = torch.randint(0, 5, (6,), generator=g)
            use_b = (i + rank) % 2 == 0                 # differs between the ranks within one microbatch
            use_side = not (step == 1 and rank == 1)
            loss = nn.functional.cross_entropy(model(x, use_b, use_side), y)
            loss.backward()
            total += loss.detach()
        if mode == "odc":
            fsdp2.pre_optimizer_step(model)
        opt.step()
        opt.zero_grad()
        dist.all_reduce(total)
        losses.append(float(total))
    full = {k: v.full_tensor().clone() for k, v in model.state_dict().items()}
    if mode == "odc":
        fsdp2.stop()
    return losses, full


@pytest.mark.parametrize("segments", ["1", "0"])
def test_fsdp2_frozen_parameters_and_skipped_branches(segments):
    a, b = run_pair(_train_partial, 2, env={"ODC_REDUCE_SEGMENTS": segments})
    assert a[0][0] == pytest.approx(b[0][0], rel=1e-5), (a[0][0], b[0][0])
    for k in a[0][1]:
        torch.testing.assert_close(a[0][1][k], b[0][1][k], rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(a[0][1]["c.weight"], b[0][1]["c.weight"], rtol=0, atol=0)  # frozen stays frozen


def _train_zero(rank, world, mode):
    """Rank 1 runs no microbatch at all in minibatches 0 and 2 (the first one included)."""
    import torch.distributed as dist
    import torch.nn as nn
    from torch.distributed.fsdp import fully_shard

    import odc_b200 as odc
    from odc_b200.fsdp import fsdp2

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(20, 32), nn.Tanh(), nn.Linear(32, 32), nn.Tanh(), nn.Linear(32, 3))
    if mode == "odc":
        odc.init_nvshmem("cpu", 64 << 20)
        fsdp2.patch_fsdp2()
    fully_shard(model[2])
    fully_shard(model)
    if mode == "odc":
        for m in (model[2], model):
            fsdp2.patch_lazy_init(m)
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    for step in range(3):
        if mode == "odc":
            fsdp2.pre_minibatch_start(model)
        idle = rank == 1 and step in (0, 2)
        for i in range(2):
            if idle and mode == "odc":
                continue  # nothing to do: no forward, no backward, no collective
            g = torch.Generator().manual_seed(100 * step + 10 * i + rank)
            x = torch.randn(5, 20, generator=g)
            y = torch.randint(0, 3, (5,), generator=g)
            loss = nn.functional.cross_entropy(model(x), y)
            (loss * (0.0 if idle else 1.0)).backward()  # lock-step FSDP has to go through the motions
        if mode == "odc":
            fsdp2.pre_optimizer_step(model)
        opt.step()
        opt.zero_grad()
    full = {k: v.full_tensor().clone() for k, v in model.state_dict().items()}
    if mode == "odc":
        fsdp2.stop()
    return full


def test_fsdp2_rank_with_zero_microbatches():
    a, b = run_pair(_train_zero, 2)
    for k in a[0]:
        torch.testing.assert_close(a[0][k], b[0][k], rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(b[0][k], b[1][k], rtol=0, atol=0)


def _train_no_sync(rank, world, mode):
    """User code written for lock-step FSDP2: gradient sync switched off for all but the last microbatch."""
    import torch.nn as nn
    from torch.distributed.fsdp import fully_shard

    import odc_b200 as odc
    from odc_b200.fsdp import fsdp2

    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(20, 32), nn.Tanh(), nn.Linear(32, 32), nn.Tanh(), nn.Linear(32, 3))
    if mode == "odc":
        odc.init_nvshmem("cpu", 64 << 20)
        fsdp2.patch_fsdp2()
    fully_shard(model[2])
    fully_shard(model)
    if mode == "odc":
        for m in (model[2], model):
            fsdp2.patch_lazy_init(m)
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    for step in range(2):
        if mode == "odc":
            fsdp2.pre_minibatch_start(model)
        for i in range(3):
            model.set_requires_gradient_sync(i == 2)
            g = torch.Generator().manual_seed(100 * step + 10 * i + rank)
            x = torch.randn(5, 20, generator=g)
            y = torch.randint(0, 3, (5,), generator=g)
            nn.functional.cross_entropy(model(x), y).backward()
        if mode == "odc":
            fsdp2.pre_optimizer_step(model)
        opt.step()
        opt.zero_grad()
    full = {k: v.full_tensor().clone() for k, v in model.state_dict().items()}
    if mode == "odc":
        fsdp2.stop()
    return full


def test_fsdp2_gradient_sync_toggle_written_for_lockstep_fsdp_still_works():
    a, b = run_pair(_train_no_sync, 2)
    for k in a[0]:
        torch.testing.assert_close(a[0][k], b[0][k], rtol=1e-5, atol=1e-6)


def _train_variants(rank, world, mode, variant):
    """Other stock FSDP2 knobs user code may carry over: no reshard after forward, explicit unshard, prefetch lists."""
    import torch.nn as nn
    from torch.distributed.fsdp import fully_shard

    import odc_b200 as odc
    from odc_b200.fsdp import fsdp2

    torch.manual_seed(0)
    blocks = [nn.Sequential(nn.Linear(24, 24), nn.Tanh()) for _ in range(3)]
    model = nn.Sequential(*blocks, nn.Linear(24, 3))
    if mode == "odc":
        odc.init_nvshmem("cpu", 64 << 20)
        fsdp2.patch_fsdp2()
    raf = variant != "keep_unsharded"
    for b in blocks:
        fully_shard(b, reshard_after_forward=raf)
    fully_shard(model, reshard_after_forward=raf)
    if variant == "prefetch":
        for i, b in enumerate(blocks):
            if i + 1 < len(blocks):
                b.set_modules_to_forward_prefetch([blocks[i + 1]])
            if i > 0:
                b.set_modules_to_backward_prefetch([blocks[i - 1]])
    if mode == "odc":
        for m in blocks + [model]:
            fsdp2.patch_lazy_init(m)
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    for step in range(2):
        if mode == "odc":
            fsdp2.pre_minibatch_start(model)
        for i in range(2):
            g = torch.Generator().manual_seed(100 * step + 10 * i + rank)
            x = torch.randn(5, 24, generator=g)
            y = torch.randint(0, 3, (5,), generator=g)
            if variant == "explicit_unshard":
                model.unshard()
            nn.functional.cross_entropy(model(x), y).backward()
        if mode == "odc":
            fsdp2.pre_optimizer_step(model)
        opt.step()
        opt.zero_grad()
    full = {k: v.full_tensor().clone() for k, v in model.state_dict().items()}
    if mode == "odc":
        fsdp2.stop()
    return full


@pytest.mark.parametrize("variant", ["keep_unsharded", "explicit_unshard", "prefetch"])
def test_fsdp2_stock_knobs_keep_working(variant):
    a, b = run_pair(_train_variants, 2, (variant,))
    for k in a[0]:
        torch.testing.assert_close(a[0][k], b[0][k], rtol=1e-5, atol=1e-6)


def _train_unused(rank, world, mode, fused):
    """In minibatch 1 no rank uses `b` (one parameter of the root group) nor the `side` unit.

    Stock FSDP leaves their ``.grad`` at None and AdamW skips them: no weight decay, no moment update.  The
    on-demand engine has to do the same, although their accumulators exist and are (all-zero) "complete".
    """
    import torch.nn as nn
    from torch.distributed.fsdp import fully_shard

    import odc_b200 as odc
    from odc_b200.fsdp import fsdp2

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.a = nn.Linear(24, 24)
            self.b = nn.Linear(24, 24)
            self.side = nn.Sequential(nn.Linear(24, 24), nn.Tanh())
            self.head = nn.Linear(24, 5)

        def forward(self, x, extras):
            h = torch.tanh(self.a(x))
            if extras:
                h = h + self.b(h)
                h = h + self.side(h)
            return self.head(h)

    torch.manual_seed(0)
    model = Net()
    if mode == "odc":
        odc.init_nvshmem("cpu", 64 << 20)
        fsdp2.patch_fsdp2()
    fully_shard(model.side)
    fully_shard(model)
    if mode == "odc":
        for m in (model.side, model):
            fsdp2.patch_lazy_init(m)
    use_fused = fused and mode == "odc"
    opt = (fsdp2.FusedAdamW(model, lr=1e-2, weight_decay=0.1) if use_fused
           else torch.optim.AdamW(model.parameters(), lr=1e-2, weight_decay=0.1))
    for step in range(3):
        if mode == "odc":
            fsdp2.pre_minibatch_start(model)
        for i in range(2):
            g = torch.Generator().manual_seed(1000 * step + 10 * i + rank)
            x = torch.randn(6, 24, generator=g)
            y = torch.randint(0, 5, (6,), generator=g)
            nn.functional.cross_entropy(model(x, extras=step != 1), y).backward()
        if mode == "odc":
            fsdp2.pre_optimizer_step(model, materialize_grads=not use_fused)
            if step == 1 and not use_fused:
                assert model.b.weight.grad is None and model.side[0].weight.grad is None
                assert model.a.weight.grad is not None
        opt.step()
        opt.zero_grad()
    full = {k: v.full_tensor().clone() for k, v in model.state_dict().items()}
    if mode == "odc":
        fsdp2.stop()
    return full


@pytest.mark.parametrize("fused", [False, True])
def test_fsdp2_parameters_no_rank_used_are_left_alone(fused):
    a, b = run_pair(_train_unused, 2, (fused,))
    for k in a[0]:
        assert_mostly_close(a[0][k], b[0][k], rtol=2e-5, atol=2e-6, outlier_atol=2e-2)
