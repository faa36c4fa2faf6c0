"""Configuration parsing, memory breakdown buckets, NVTX shims and the clock sampler's parser (pure CPU)."""
import os
import stat
import textwrap

import pytest
import torch


def test_parse_size_and_env_overrides(monkeypatch):
    from odc_b200 import config
    assert config.parse_size("5G") == 5 << 30 and config.parse_size("512m") == 512 << 20
    assert config.parse_size("1073741824") == 1 << 30 and config.parse_size("2GiB") == 2 << 30
    monkeypatch.delenv("ODC_SYMMETRIC_SIZE", raising=False)
    monkeypatch.setenv("NVSHMEM_SYMMETRIC_SIZE", "30G")         # launch scripts written for the reference keep working
    assert config.symmetric_size("cuda") == 30 << 30
    monkeypatch.setenv("ODC_SYMMETRIC_SIZE", "10G")
    assert config.symmetric_size("cuda") == 10 << 30
    monkeypatch.setenv("RAY_LOCAL_WORLD_SIZE", "4")
    monkeypatch.setenv("LOCAL_WORLD_SIZE", "8")
    assert config.local_world_size(16) == 4                      # the Ray variable wins
    monkeypatch.setenv("ODC_WAIT_TIMEOUT_MS", "123")
    assert config.wait_timeout_ms() == 123


def test_memory_breakdown_buckets_single_rank():
    import odc_b200 as odc
    from odc_b200.fsdp import fsdp2
    reg = odc.init_nvshmem("cpu", 64 << 20)
    try:
        reg.allocate_symm_buffer("fsdp_params_gather_0", (1 << 18,), torch.float32)
        reg.allocate_symm_buffer("fsdp_params_lowp_fsdp_params_gather_0", (1 << 18,), torch.bfloat16)
        reg.allocate_symm_buffer("hpz_fsdp_params_gather_0", (1 << 18,), torch.bfloat16)
        reg.allocate_symm_buffer("rs_accumulation_0", (1 << 18,), torch.float32)
        reg.allocate_symm_buffer("something_else", (1 << 10,), torch.int32)
        b = fsdp2.get_symm_buffer_memory_breakdown()
        assert b["fsdp_params"] == pytest.approx(1.0 / 1024) and b["accumulation"] == pytest.approx(1.0 / 1024)
        assert b["lowp_replica"] == pytest.approx(0.5 / 1024) and b["hpz_buffer"] == pytest.approx(0.5 / 1024)
        assert b["other"] > 0 and b["total"] == pytest.approx(sum(v for k, v in b.items() if k != "total"))
        assert reg.memory_allocated() == sum(reg.memory_by_key().values())
        # registry semantics: reverse lookup, epoch flush
        w = reg.get_symm_buffer("something_else")
        assert reg.key_of(w)[0] == "something_else" and reg.has_key("something_else")
        v = torch.arange(1 << 10, dtype=torch.int32)
        reg.update_symm_buffer("something_else", v)
        reg.update_symm_buffer("something_else", v + 1)           # same epoch: not copied again
        assert torch.equal(w, v)
        reg.flush()
        reg.update_symm_buffer("something_else", v + 1)
        assert torch.equal(w, v + 1)
        reg.deallocate_symm_buffer("something_else")
        assert not reg.has_key("something_else")
    finally:
        odc.finalize_distributed()


def test_nvtx_helpers_are_noops_without_cuda():
    from odc_b200.utils import nvtx_range, nvtx_record_function
    with nvtx_range("x"):
        pass
    with nvtx_record_function("y"):
        pass


def test_clock_sampler_parses_nvidia_smi_output(tmp_path, monkeypatch):
    """A fake nvidia-smi on PATH prints CSV rows; the sampler reports the median clock under load and the reasons."""
    fake = tmp_path / "nvidia-smi"
    fake.write_text(textwrap.dedent("""\
        #!/bin/sh
        echo "0, 1900, 1965, 300.0, 0x0, Not Active, Not Active, Not Active, Not Active"
        echo "0, 1350, 1965, 990.0, 0x4, Not Active, Not Active, Not Active, Active"
        echo "0, 1370, 1965, 1001.0, 0x4, Not Active, Not Active, Not Active, Active"
        sleep 5
    """))
    fake.chmod(fake.stat().st_mode | stat.S_IEXEC)
    monkeypatch.setenv("PATH", f"{tmp_path}:{os.environ['PATH']}")
    from odc_b200.utils.clocks import ClockSampler
    import time
    s = ClockSampler(gpu_index=0).start()
    deadline = time.time() + 20.0           # the fake tool prints its three rows at once; wait until they are on disk
    while time.time() < deadline and sum(1 for _ in open(s.path)) < 3:
        time.sleep(0.05)
    out = s.stop()
    assert out["samples"] == 3 and out["sm_max_mhz"] == 1965.0
    assert out["sm_mhz"] == pytest.approx(1360.0)                 # median of the samples taken under load
    assert out["reasons"] == ["sw_power_cap"]


def test_inter_node_transport_needs_a_multi_node_job():
    import odc_b200 as odc
    from odc_b200.runtime import InterNodeTransport
    reg = odc.init_nvshmem("cpu", 1 << 20)  # single process: one node, no endpoint is started
    try:
        assert reg.internode is None
        with pytest.raises(RuntimeError):
            InterNodeTransport(reg)
    finally:
        odc.finalize_distributed()


def test_linear_token_logprobs_cpu_matches_plain_autograd():
    """The chunked per-token log-probability head (policy-gradient losses) equals log_softmax + gather, with a
    temperature, ignored positions, a 3-D input and a ragged last chunk; the module form returns (log_probs, None)."""
    from odc_b200 import ops
    torch.manual_seed(0)
    B, S, H, V = 2, 37, 16, 50
    h = torch.randn(B, S, H, requires_grad=True)
    w = torch.randn(V, H, requires_grad=True)
    ids = torch.randint(0, V, (B, S))
    ids[1, 3] = -100
    adv = torch.randn(B, S)
    lp, ent = ops.LinearTokenLogProbs(chunk_size=16)(h, w, ids, temperature=0.5)
    assert ent is None and lp.shape == (B, S)
    (lp * adv).sum().backward()
    h2, w2 = h.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    full = ((h2 @ w2.t()) / 0.5).log_softmax(-1).gather(-1, ids.clamp_min(0).unsqueeze(-1)).squeeze(-1)
    full = torch.where(ids != -100, full, torch.zeros_like(full))
    (full * adv).sum().backward()
    torch.testing.assert_close(lp, full.detach())
    torch.testing.assert_close(h.grad, h2.grad)
    torch.testing.assert_close(w.grad, w2.grad)
    assert float(lp.detach()[1, 3]) == 0.0 and float(h.grad[1, 3].abs().max()) == 0.0


def test_decoder_logprob_head_gives_the_same_loss_and_gradients():
    """``DecoderLM(..., return_logprobs=True)`` weighted by ``loss_scale`` is the fused cross-entropy loss."""
    from odc_b200.data import LengthSpec, make_minibatch
    from odc_b200.models import DecoderConfig, DecoderLM
    cfg = DecoderConfig(vocab_size=97, hidden_size=32, intermediate_size=64, num_layers=1, num_heads=2, num_kv_heads=1,
                        head_dim=16)
    mb = make_minibatch(0, 0, cfg.vocab_size, LengthSpec("uniform", lo=8, hi=40), 1, 128)[0]
    a = (mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"])
    grads = []
    losses = []
    for head in ("ce", "logprobs"):
        model = DecoderLM(cfg)
        model.reset_parameters(seed=1)
        if head == "ce":
            loss = model(*a, labels=mb["labels"], loss_scale=mb["loss_scale"])
        else:
            loss = -(model(*a, labels=mb["labels"], return_logprobs=True) * mb["loss_scale"]).sum()
        loss.backward()
        losses.append(loss.detach())
        grads.append({n: p.grad.clone() for n, p in model.named_parameters()})
    torch.testing.assert_close(losses[0], losses[1])
    for n in grads[0]:
        torch.testing.assert_close(grads[0][n], grads[1][n], rtol=1e-4, atol=1e-6)
