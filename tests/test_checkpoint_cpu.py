"""Checkpoint round trips between the on-demand engine and stock FSDP2 (CPU/gloo, world 2)."""
import os
import tempfile

import pytest
import torch

from _mp import assert_mostly_close, run_ranks


def _build(mode, mesh):
    from torch.distributed.fsdp import fully_shard

    from odc_b200.fsdp import fsdp2
    from odc_b200.models import DecoderLM, get_config
    model = DecoderLM(get_config("tiny"))
    model.reset_parameters(seed=1 if mode == "odc" else 2)  # different inits: loading must overwrite them
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    return model


def _one_step(model, rank, odc_mode):
    from odc_b200.data import LengthSpec, make_minibatch
    from odc_b200.fsdp import fsdp2
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    if odc_mode:
        fsdp2.pre_minibatch_start(model)
    mb = make_minibatch(rank, 0, 1024, LengthSpec("uniform", lo=16, hi=64), 1, 64, seed=3)[0]
    loss = model(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"], labels=mb["labels"],
                 loss_scale=mb["loss_scale"])
    loss.backward()
    if odc_mode:
        fsdp2.pre_optimizer_step(model)
    opt.step(); opt.zero_grad()
    return opt, float(loss)


def _roundtrip(rank, world, folder, dcp_api, direction):
    import torch.distributed as dist
    import torch.distributed.checkpoint as dcp
    from torch.distributed.device_mesh import init_device_mesh

    import odc_b200 as odc
    from odc_b200.fsdp import fsdp2
    from odc_b200.utils.checkpoint import Checkpointer
    mesh = init_device_mesh("cpu", (world,))
    odc.init_nvshmem("cpu", 256 << 20)
    src_odc = direction == "odc_to_stock"
    # ---- writer
    if src_odc:
        fsdp2.patch_fsdp2()
    writer = _build("odc" if src_odc else "stock", mesh)
    if src_odc:
        for m in list(writer.layers) + [writer]:
            fsdp2.patch_lazy_init(m)
    opt, _ = _one_step(writer, rank, src_odc)
    ck = Checkpointer(folder, dcp_api=dcp_api)
    ck.save(writer, opt)
    sharded_dir = os.path.join(folder, "sharded")
    dcp.save({"model": writer.state_dict()}, checkpoint_id=sharded_dir)  # sharded DCP layout, as stock FSDP2 writes it
    want = {k: v.full_tensor().clone() for k, v in writer.state_dict().items()}
    if src_odc:
        fsdp2.unpatch_fsdp2()
    # ---- reader (the other engine)
    if not src_odc:
        fsdp2.patch_fsdp2()
    reader = _build("stock" if src_odc else "odc", mesh)
    ck2 = Checkpointer(folder, dcp_api=dcp_api)
    assert not ck2.is_empty()
    ck2.load_model(reader)                      # before lazy init: weights are copied into the heap at first use
    if not src_odc:
        for m in list(reader.layers) + [reader]:
            fsdp2.patch_lazy_init(m)
    got = {k: v.full_tensor().clone() for k, v in reader.state_dict().items()}
    for k in want:
        assert torch.equal(want[k], got[k]), k
    # sharded DCP load into the reader as well
    for p in reader.parameters():
        p.data.zero_()
    sd = {"model": reader.state_dict()}
    dcp.load(sd, checkpoint_id=sharded_dir)
    got = {k: v.full_tensor().clone() for k, v in reader.state_dict().items()}
    for k in want:
        assert torch.equal(want[k], got[k]), k
    # the loaded model trains, and under the on-demand engine its parameters sit in the heap
    opt2, loss = _one_step(reader, rank, not src_odc)
    assert loss == loss
    if not src_odc:
        reg = odc.SymmBufferRegistry.get_instance()
        p0 = next(reader.parameters())
        assert reg.heap.offset_of(p0._local_tensor) is not None
        # a later assign=True load detaches parameters from the heap; repin puts them back
        full = {k: v.full_tensor() for k, v in reader.state_dict().items()}
        from torch.distributed.checkpoint.state_dict import StateDictOptions, set_model_state_dict
        set_model_state_dict(reader, full, options=StateDictOptions(full_state_dict=True))
        fsdp2.repin_sharded_params(reader)
        assert reg.heap.offset_of(next(reader.parameters())._local_tensor) is not None
        _one_step(reader, rank, True)
        fsdp2.stop()
    else:
        odc.finalize_distributed()
    return True


@pytest.mark.parametrize("dcp_api", [True, False])
@pytest.mark.parametrize("direction", ["odc_to_stock", "stock_to_odc"])
def test_checkpoint_roundtrip(dcp_api, direction):
    with tempfile.TemporaryDirectory() as folder:
        assert all(run_ranks(_roundtrip, 2, folder, dcp_api, direction))


def _tiny(mesh, seed):
    from torch.distributed.fsdp import fully_shard

    from odc_b200.models import DecoderLM, get_config
    model = DecoderLM(get_config("tiny"))
    model.reset_parameters(seed=seed)
    for layer in model.layers:
        fully_shard(layer, mesh=mesh)
    fully_shard(model, mesh=mesh)
    return model


def _minibatch(model, opt, rank, step, engine_on, fused):
    from odc_b200.data import LengthSpec, make_minibatch
    from odc_b200.fsdp import fsdp2
    if engine_on:
        fsdp2.pre_minibatch_start(model)
    for mb in make_minibatch(rank, step, 1024, LengthSpec("uniform", lo=16, hi=64), 2, 64, seed=5):
        model(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"], labels=mb["labels"],
              loss_scale=mb["loss_scale"]).backward()
    if engine_on:
        fsdp2.pre_optimizer_step(model, materialize_grads=not fused)
    opt.step()
    opt.zero_grad()


def _resume(rank, world, folder, writer_kind, reader_kind):
    """Write after two minibatches, resume in a fresh model with the same or the other optimizer / engine."""
    from torch.distributed.device_mesh import init_device_mesh

    import odc_b200 as odc
    from odc_b200.fsdp import fsdp2
    from odc_b200.utils.checkpoint import Checkpointer
    mesh = init_device_mesh("cpu", (world,))
    odc.init_nvshmem("cpu", 256 << 20)

    def make(kind, seed):
        on = kind == "fused"
        if on:
            fsdp2.patch_fsdp2()
        else:
            fsdp2.unpatch_fsdp2()
        model = _tiny(mesh, seed)
        if on:
            for m in list(model.layers) + [model]:
                fsdp2.patch_lazy_init(m)
        opt = (fsdp2.FusedAdamW(model, lr=2e-3, weight_decay=0.05) if on
               else torch.optim.AdamW(model.parameters(), lr=2e-3, weight_decay=0.05))
        return model, opt, on

    model, opt, on = make(writer_kind, 1)
    for step in range(2):
        _minibatch(model, opt, rank, step, on, on)
    ck = Checkpointer(folder)
    ck.save(model, opt)
    _minibatch(model, opt, rank, 2, on, on)          # the uninterrupted run
    want = {k: v.full_tensor().clone() for k, v in model.state_dict().items()}

    model2, opt2, on2 = make(reader_kind, 2)         # different initial weights: the load must replace them
    ck2 = Checkpointer(folder)
    ck2.load_model(model2)
    ck2.load_optim(model2, opt2)
    _minibatch(model2, opt2, rank, 2, on2, on2)
    got = {k: v.full_tensor().clone() for k, v in model2.state_dict().items()}
    if on2:
        fsdp2.stop()
    return want, got


@pytest.mark.parametrize("writer,reader", [("fused", "fused"), ("fused", "torch"), ("torch", "fused")])
def test_resume_with_fused_or_torch_adamw(writer, reader):
    with tempfile.TemporaryDirectory() as folder:
        want, got = run_ranks(_resume, 2, folder, writer, reader)[0]
    for k in want:
        assert_mostly_close(got[k], want[k], rtol=1e-5, atol=1e-6, outlier_atol=4e-3)
