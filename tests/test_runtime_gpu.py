"""Symmetric heap, services and the FSDP2 path on one GPU (world size 1)."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture()
def single_rank_pg():
    import torch.distributed as dist
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    created = False
    if not dist.is_initialized():
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
        created = True
    yield
    if created:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["vmm", "ipc"])
def test_heap_and_services_world1(mode, monkeypatch):
    import odc_b200 as odc
    monkeypatch.setenv("ODC_HEAP_MODE", mode)
    monkeypatch.setenv("ODC_IPC_SLAB_SIZE", "1G")
    torch.cuda.set_device(0)
    reg = odc.init_nvshmem(torch.device("cuda", 0), 4 << 30)
    try:
        assert reg.heap.mode == mode
        a = reg.allocate_symm_buffer("a", (1 << 20,), torch.float32)
        b = reg.allocate_symm_buffer("b", (300 << 20,), torch.bfloat16)  # forces a second growth step in vmm mode
        a.copy_(torch.arange(1 << 20, device="cuda", dtype=torch.float32))
        b.fill_(1.5)
        assert float(b.float().sum()) == 1.5 * (300 << 20)
        g = odc.GatherService()
        out = torch.empty(1 << 20, dtype=torch.bfloat16, device="cuda")
        g.gather_into_tensor(out, a)
        assert torch.equal(out, a.bfloat16())
        red = odc.ReductionService(accumulation_dtype=torch.float32)
        x = torch.randint(-3, 4, (1 << 16,), device="cuda").bfloat16()
        red.scatter_accumulate("k", x)
        red.scatter_accumulate("k", x)
        red.sync()
        assert torch.equal(red.get_accumulation("k"), 2 * x.float())
        assert reg.memory_allocated() >= (1 << 22) + (600 << 20)
        red.stop()
    finally:
        odc.finalize_distributed()


def test_ipc_handle_roundtrip():
    from odc_b200 import _ext
    ext = _ext.load()
    t = torch.arange(1024, device="cuda", dtype=torch.float32)
    blob = ext.get_ipc_handle(t[16:])
    assert isinstance(blob, bytes) and len(blob) == 64 + 8


def test_fsdp2_single_gpu_training_step(single_rank_pg, monkeypatch):
    """Tiny decoder, FSDP2 world 1, on-demand path + fused optimizer: loss goes down, grads land in the accumulators."""
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    import odc_b200 as odc
    from odc_b200.data import LengthSpec, make_minibatch, to_device
    from odc_b200.fsdp import fsdp2
    from odc_b200.models import DecoderLM, get_config

    dev = torch.device("cuda", 0)
    cfg = get_config("tiny")
    with torch.device(dev):
        model = DecoderLM(cfg)
    model.reset_parameters(seed=0)
    odc.init_nvshmem(dev, 2 << 30)
    fsdp2.patch_fsdp2()
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    for layer in model.layers:
        fully_shard(layer, mp_policy=mp)
    fully_shard(model, mp_policy=mp)
    for m in list(model.layers) + [model]:
        fsdp2.patch_lazy_init(m)
    opt = fsdp2.FusedAdamW(model, lr=3e-3)
    mbs = [to_device(mb, dev) for mb in make_minibatch(0, 0, cfg.vocab_size, LengthSpec("uniform", lo=16, hi=128), 2, 512)]
    losses = []
    try:
        for step in range(6):
            fsdp2.pre_minibatch_start(model)
            tot = 0.0
            for mb in mbs:
                loss = model(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"],
                             labels=mb["labels"], loss_scale=mb["loss_scale"])
                loss.backward()
                tot += float(loss)
            fsdp2.pre_optimizer_step(model, materialize_grads=False)
            norm = opt.clip_grad_norm_(1.0)
            assert torch.isfinite(norm)
            opt.step()
            opt.zero_grad()
            losses.append(tot)
        assert losses[-1] < losses[0] - 0.05, losses
        assert fsdp2.transport_launches() > 0
    finally:
        fsdp2.stop()


@pytest.mark.parametrize("head", ["ce", "logprobs"])
def test_fused_engine_single_gpu_training_step(single_rank_pg, head):
    """Tiny decoder on the fused-kernel engine, world 1: the loss goes down with either LM head, the clip norm is
    finite, and the whole-model state has ``DecoderLM``'s names."""
    import odc_b200 as odc
    from odc_b200.data import LengthSpec, make_minibatch, to_device
    from odc_b200.models import DecoderLM, get_config
    from odc_b200.parallel import FusedDecoderLM, FusedOptimizer

    dev = torch.device("cuda", 0)
    cfg = get_config("tiny")
    odc.init_nvshmem(dev, 2 << 30)
    model = FusedDecoderLM(cfg, device=dev, seed=0)
    opt = FusedOptimizer(model, lr=3e-3)
    mbs = [to_device(mb, dev) for mb in make_minibatch(0, 0, cfg.vocab_size, LengthSpec("uniform", lo=16, hi=128), 2, 512)]
    losses = []
    try:
        for step in range(6):
            model.start_minibatch()
            tot = 0.0
            for mb in mbs:
                a = (mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"])
                if head == "ce":
                    loss = model(*a, labels=mb["labels"], loss_scale=mb["loss_scale"])
                else:
                    loss = -(model(*a, labels=mb["labels"], return_logprobs=True) * mb["loss_scale"]).sum()
                loss.backward()
                tot += float(loss.detach())
            model.finish_minibatch()
            assert torch.isfinite(opt.clip_grad_norm_(1.0))
            opt.step()
            losses.append(tot)
        assert losses[-1] < losses[0] - 0.05, losses
        with torch.device("meta"):
            names = set(DecoderLM(cfg).state_dict())
        assert set(model.full_state_dict()) == names
    finally:
        model.stop()


def test_deterministic_reduction_mode_gpu(monkeypatch):
    import odc_b200 as odc
    monkeypatch.setenv("ODC_DETERMINISTIC", "1")
    torch.cuda.set_device(0)
    odc.init_nvshmem(torch.device("cuda", 0), 1 << 30)
    try:
        red = odc.ReductionService(accumulation_dtype=torch.float32)
        assert red.deterministic
        xs = [torch.randn(1 << 16, device="cuda") for _ in range(3)]
        for x in xs:
            red.scatter_accumulate("k", x)
        red.sync()
        want = torch.zeros(1 << 16, device="cuda")
        for x in xs:
            want += x
        assert torch.equal(red.get_accumulation("k"), want)
        red.stop()
    finally:
        odc.finalize_distributed()


def test_pipeline_status_surfaces_at_the_next_sync(single_rank_pg):
    """A GEMM / attention pipeline wait that ran out is recorded in the device's status word; the communication
    service reads that same word at every synchronisation point and raises.  The word is pre-set here by hand:
    nothing on the GPU is made to stall."""
    import odc_b200 as odc
    from odc_b200 import _ext
    from odc_b200.runtime.status import ERR_PIPELINE_TIMEOUT, OdcTimeoutError
    torch.cuda.set_device(0)
    odc.init_nvshmem(torch.device("cuda", 0), 1 << 30)
    try:
        red = odc.ReductionService(accumulation_dtype=torch.float32)
        x = torch.ones(1 << 12, device="cuda")
        red.scatter_accumulate("k", x)
        red.sync()                                   # clean
        word = _ext.load().kernel_status()
        assert word.data_ptr() == red.transport.status.data_ptr()
        word.copy_(torch.tensor([ERR_PIPELINE_TIMEOUT, 3, 17, 0], dtype=torch.int32))
        red.scatter_accumulate("k", x)
        with pytest.raises(OdcTimeoutError, match="pipeline"):
            red.sync()
        assert int(word[0]) == 0                     # reported once, then cleared
        red.scatter_accumulate("k", x)
        red.sync()
        assert float(red.get_accumulation("k").sum()) == 3 * (1 << 12)
        red.stop()
    finally:
        odc.finalize_distributed()
