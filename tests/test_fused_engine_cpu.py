"""The fused-kernel decoder engine (``parallel.FusedDecoderLM``) against stock FSDP2 on CPU ranks (gloo)."""
import os

import pytest
import torch

from _mp import assert_mostly_close, run_pair


def _make_batches(rank, step, n_micro, vocab=1024):
    from odc_b200.data import LengthSpec, make_minibatch
    return make_minibatch(rank, step, vocab, LengthSpec("uniform", lo=16, hi=128), n_micro, 128, seed=7)


def _train(rank, world, mode, steps, uneven, variant):
    import torch.distributed as dist
    from torch.distributed.fsdp import fully_shard

    import odc_b200 as odc
    from odc_b200.models import DecoderLM, get_config
    from odc_b200.parallel import FusedDecoderLM, FusedOptimizer

    over = {}
    if "bias_tied" in variant:
        over.update(qkv_bias=True, tie_embeddings=True)
    if "ac" in variant:
        over.update(activation_checkpointing=True)
    cfg = get_config("tiny", **over)
    torch.manual_seed(0)
    if mode == "stock":
        model = DecoderLM(cfg)
        model.reset_parameters(seed=0)
        if cfg.qkv_bias:   # zero biases would hide a wrong bias gradient
            with torch.no_grad():
                for layer in model.layers:
                    layer.attn.bqkv.normal_(0, 0.02, generator=torch.Generator().manual_seed(5))
        for layer in model.layers:
            fully_shard(layer)
        fully_shard(model)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    else:
        odc.init_nvshmem("cpu", 256 << 20)
        src = DecoderLM(cfg)
        src.reset_parameters(seed=0)
        if cfg.qkv_bias:
            with torch.no_grad():
                for layer in src.layers:
                    layer.attn.bqkv.normal_(0, 0.02, generator=torch.Generator().manual_seed(5))
        model = FusedDecoderLM(cfg, device="cpu", source=src, keep_weight="keep" in variant)
        opt = FusedOptimizer(model, lr=1e-3)
    losses = []
    for step in range(steps):
        if mode == "odc":
            model.start_minibatch()
        mine = (2 + rank) if uneven else 2
        n_micro = mine
        if uneven and mode == "stock":
            n_micro = 2 + world - 1      # lock-step FSDP must run the same count: pad with zero-weight work
        total = torch.zeros(())
        for i in range(n_micro):
            real = i < mine
            mb = _make_batches(rank, step, mine)[i if real else 0]
            if mode == "odc" and "defer" in variant:
                model.set_requires_gradient_sync(i == n_micro - 1)
            a = (mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"])
            if mode == "odc" and "logprobs" in variant:   # the per-token log-probability head gives the same loss
                loss = -(model(*a, labels=mb["labels"], return_logprobs=True) * mb["loss_scale"]).sum()
            else:
                loss = model(*a, labels=mb["labels"], loss_scale=mb["loss_scale"])
            if not real:
                loss = loss * 0.0
            loss.backward()
            total += loss.detach()
        if mode == "odc":
            model.finish_minibatch()
            if "clip" in variant:
                opt.clip_grad_norm_(0.5)
        elif "clip" in variant:
            torch.nn.utils.clip_grad_norm_(model.parameters(), 0.5)
        opt.step()
        opt.zero_grad()
        dist.all_reduce(total)
        losses.append(float(total))
    if mode == "stock":
        full = {k: v.full_tensor().clone() for k, v in model.state_dict().items()}
    else:
        full = model.full_state_dict()
        if "roundtrip" in variant:   # whole-model state out and back in: nothing changes
            osd = opt.full_state_dict()
            model.load_full_state_dict(full)
            opt.load_full_state_dict(osd)
            again = model.full_state_dict()
            assert all(torch.equal(full[k], again[k]) for k in full)
            assert torch.equal(opt.full_state_dict()["exp_avg"]["norm.weight"], osd["exp_avg"]["norm.weight"])
        model.stop()
    return losses, full


@pytest.mark.parametrize("uneven,variant", [(False, "plain,roundtrip"), (True, "defer,clip,logprobs"),
                                            (False, "bias_tied,keep,ac"), (True, "bias_tied,defer,logprobs")])
def test_fused_engine_matches_stock_fsdp2(uneven, variant):
    world = 2
    a, b = run_pair(_train, world, (3, uneven, variant))
    la, lb = a[0][0], b[0][0]
    assert la == pytest.approx(lb, rel=1e-4), (la, lb)
    assert set(a[0][1]) == set(b[0][1])
    for k in a[0][1]:
        assert a[0][1][k].shape == b[0][1][k].shape, k
        assert_mostly_close(b[0][1][k], a[0][1][k], rtol=5e-3, atol=2e-4)


def _checkpoint_roundtrip(rank, world, folder):
    """A model + optimizer checkpoint written under stock FSDP2 continues on the fused engine, and back."""
    import torch.distributed as dist
    from torch.distributed.fsdp import fully_shard

    import odc_b200 as odc
    from odc_b200.models import DecoderLM, get_config
    from odc_b200.parallel import FusedDecoderLM, FusedOptimizer
    from odc_b200.utils.checkpoint import Checkpointer

    cfg = get_config("tiny")
    mb = _make_batches(rank, 0, 1)[0]

    def loss_of(m):
        return m(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"], labels=mb["labels"],
                 loss_scale=mb["loss_scale"])

    # stock FSDP2: one optimizer step, save
    stock = DecoderLM(cfg)
    stock.reset_parameters(seed=3)
    for layer in stock.layers:
        fully_shard(layer)
    fully_shard(stock)
    opt = torch.optim.AdamW(stock.parameters(), lr=1e-3)
    loss_of(stock).backward()
    opt.step(); opt.zero_grad()
    ck = Checkpointer(folder)
    ck.save(stock, opt)
    with torch.no_grad():
        want = float(loss_of(stock))

    # fused engine: other initial weights, load, same loss; then take a step on both and compare the weights
    odc.init_nvshmem("cpu", 256 << 20)
    fused = FusedDecoderLM(cfg, device="cpu", seed=9)
    fopt = FusedOptimizer(fused, lr=1e-3)
    ck2 = Checkpointer(folder)
    ck2.load_model(fused)
    ck2.load_optim(fused, fopt)
    fused.start_minibatch()
    loss = loss_of(fused)
    got = float(loss.detach())
    loss.backward()
    fused.finish_minibatch()
    fopt.step()
    loss_of(stock).backward()
    opt.step(); opt.zero_grad()
    a = {k: v.full_tensor() for k, v in stock.state_dict().items()}
    b = fused.full_state_dict()
    close = all(torch.allclose(a[k], b[k], rtol=5e-3, atol=2e-4) for k in a)
    # and back: the fused engine's file loads into a fresh stock model
    folder2 = os.path.join(folder, "from_fused")
    Checkpointer(folder2).save(fused, fopt)
    fresh = DecoderLM(cfg)
    fresh.reset_parameters(seed=11)
    for layer in fresh.layers:
        fully_shard(layer)
    fully_shard(fresh)
    Checkpointer(folder2).load_model(fresh)
    c = {k: v.full_tensor() for k, v in fresh.state_dict().items()}
    back = all(torch.equal(b[k], c[k]) for k in b)
    dist.barrier()
    fused.stop()
    return want, got, close, back


def test_checkpoint_moves_between_stock_fsdp2_and_fused_engine(tmp_path):
    from _mp import run_ranks
    res = run_ranks(_checkpoint_roundtrip, 2, str(tmp_path))
    for want, got, close, back in res:
        assert got == pytest.approx(want, rel=1e-5)
        assert close and back


def _train_hsdp(rank, world, mode):
    """Hybrid sharding, 2 replicas x 2 shards: stock FSDP2 on a 2-D mesh against the fused engine on the same mesh."""
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    import odc_b200 as odc
    from odc_b200.models import DecoderLM, get_config
    from odc_b200.parallel import FusedDecoderLM, FusedOptimizer

    cfg = get_config("tiny")
    mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("dp_replicate", "dp_shard"))
    if mode == "stock":
        model = DecoderLM(cfg)
        model.reset_parameters(seed=0)
        for layer in model.layers:
            fully_shard(layer, mesh=mesh)
        fully_shard(model, mesh=mesh)
        opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    else:
        odc.init_nvshmem("cpu", 256 << 20)
        model = FusedDecoderLM(cfg, device="cpu", seed=0, mesh=mesh)
        opt = FusedOptimizer(model, lr=1e-3)
    losses = []
    for step in range(3):
        if mode == "odc":
            model.start_minibatch()
        mine = 1 + rank % 3                       # 1, 2, 3, 1 microbatches
        n_micro = mine if mode == "odc" else 3
        total = torch.zeros(())
        for i in range(n_micro):
            real = i < mine
            mb = _make_batches(rank, step, mine)[i if real else 0]
            loss = model(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"],
                         labels=mb["labels"], loss_scale=mb["loss_scale"])
            loss = loss if real else loss * 0.0
            loss.backward()
            total += loss.detach()
        if mode == "odc":
            model.finish_minibatch()
            opt.clip_grad_norm_(0.5)
        else:
            torch.nn.utils.clip_grad_norm_(model.parameters(), 0.5)
        opt.step()
        opt.zero_grad()
        dist.all_reduce(total)
        losses.append(float(total))
    if mode == "stock":
        full = {k: v.full_tensor().clone() for k, v in model.state_dict().items()}
    else:
        full = model.full_state_dict()
        model.stop()
    return losses, full


def test_fused_engine_hybrid_sharding_matches_stock_hsdp():
    a, b = run_pair(_train_hsdp, 4)
    assert a[0][0] == pytest.approx(b[0][0], rel=1e-4), (a[0][0], b[0][0])
    for r in (0, 3):   # a rank of each replica
        for k in a[r][1]:
            assert_mostly_close(b[r][1][k], a[r][1][k], rtol=5e-3, atol=2e-4)


def _save_small(rank, world, folder):
    import odc_b200 as odc
    from odc_b200.models import get_config
    from odc_b200.parallel import FusedDecoderLM, FusedOptimizer
    from odc_b200.utils.checkpoint import Checkpointer
    odc.init_nvshmem("cpu", 256 << 20)
    model = FusedDecoderLM(get_config("tiny"), device="cpu", seed=1)
    opt = FusedOptimizer(model, lr=1e-3)
    mb = _make_batches(rank, 0, 1)[0]
    model.start_minibatch()
    model(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"], labels=mb["labels"],
          loss_scale=mb["loss_scale"]).backward()
    model.finish_minibatch()
    opt.step()
    Checkpointer(folder).save(model, opt, meta={"next_step": 1})
    model.stop()
    return True


def _load_small(rank, world, folder):
    import odc_b200 as odc
    from odc_b200.models import get_config
    from odc_b200.parallel import FusedDecoderLM, FusedOptimizer
    from odc_b200.utils.checkpoint import MODEL_FILE, OPTIM_FILE, Checkpointer
    odc.init_nvshmem("cpu", 256 << 20)
    model = FusedDecoderLM(get_config("tiny"), device="cpu", seed=2)
    opt = FusedOptimizer(model, lr=1e-3)
    ck = Checkpointer(folder)
    ck.load_model(model)
    ck.load_optim(model, opt)
    saved = torch.load(os.path.join(folder, ck.last_training_time, MODEL_FILE), weights_only=True)
    saved_opt = torch.load(os.path.join(folder, ck.last_training_time, OPTIM_FILE), weights_only=True)
    now, now_opt = model.full_state_dict(), opt.full_state_dict()
    same = all(torch.equal(now[k], saved[k]) for k in saved) and ck.load_meta() == {"next_step": 1}
    same_opt = all(torch.equal(now_opt["exp_avg"][k], saved_opt["exp_avg"][k]) for k in saved_opt["exp_avg"])
    # and the resharded job trains on
    mb = _make_batches(rank, 1, 1)[0]
    model.start_minibatch()
    loss = model(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"], labels=mb["labels"],
                 loss_scale=mb["loss_scale"])
    loss.backward()
    model.finish_minibatch()
    opt.step()
    model.stop()
    return same, same_opt, float(loss.detach())


def test_checkpoint_written_on_two_ranks_resumes_on_three(tmp_path):
    """Checkpoints hold whole tensors, so a job can come back with a different number of ranks (rows are re-split)."""
    from _mp import run_ranks
    assert all(run_ranks(_save_small, 2, str(tmp_path)))
    for same, same_opt, loss in run_ranks(_load_small, 3, str(tmp_path)):
        assert same and same_opt and loss == loss
