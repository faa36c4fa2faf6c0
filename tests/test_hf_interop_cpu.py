"""Hugging Face Llama / Qwen2 checkpoints convert to this decoder and back: same logits, same tensors (pure CPU)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def _tiny(kind):
    if kind == "llama3_scaled":   # Llama 3.1 / 3.2: rescaled rotary frequencies; 16 original positions put the 8
        # frequencies of a 16-wide head into all three bands of the rule
        conf = transformers.LlamaConfig(vocab_size=211, hidden_size=64, intermediate_size=112, num_hidden_layers=2,
                                        num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-5,
                                        tie_word_embeddings=True,
                                        rope_parameters={"rope_type": "llama3", "rope_theta": 10000.0, "factor": 8.0,
                                                         "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                                                         "original_max_position_embeddings": 16})
        cls = transformers.LlamaForCausalLM
    elif kind == "llama":
        conf = transformers.LlamaConfig(vocab_size=211, hidden_size=64, intermediate_size=112, num_hidden_layers=2,
                                        num_attention_heads=4, num_key_value_heads=2, rms_norm_eps=1e-5,
                                        rope_theta=50000.0, tie_word_embeddings=False)
        cls = transformers.LlamaForCausalLM
    else:
        conf = transformers.Qwen2Config(vocab_size=211, hidden_size=64, intermediate_size=112, num_hidden_layers=2,
                                        num_attention_heads=4, num_key_value_heads=1, rms_norm_eps=1e-6,
                                        rope_theta=1000000.0, tie_word_embeddings=True)
        cls = transformers.Qwen2ForCausalLM
    conf._attn_implementation = "eager"
    torch.manual_seed(0)
    model = cls(conf).float().eval()
    with torch.no_grad():
        for n, p in model.named_parameters():
            if n.endswith("bias") or "layernorm" in n or n.endswith("norm.weight"):
                p.add_(0.1 * torch.randn_like(p))   # zero biases / unit norm weights would hide a misplaced tensor
    return conf, model


@pytest.mark.parametrize("kind", ["llama", "qwen2", "llama3_scaled"])
def test_hf_checkpoint_gives_the_same_logits(kind, tmp_path):
    from odc_b200.models import DecoderLM
    from odc_b200.models import hf
    conf, hf_model = _tiny(kind)
    cfg = hf.config_from_hf(conf)
    assert cfg.qkv_bias == (kind == "qwen2") and cfg.tie_embeddings == (kind != "llama")
    assert cfg.head_dim == 16 and cfg.num_kv_heads == (1 if kind == "qwen2" else 2)
    assert (cfg.rope_scaling is not None) == (kind == "llama3_scaled")
    sd = hf.state_dict_from_hf(hf_model.state_dict(), cfg)
    model = DecoderLM(cfg)
    model.load_state_dict(sd)
    T = 23
    ids = torch.randint(0, cfg.vocab_size, (T,))
    with torch.no_grad():
        want = hf_model(input_ids=ids[None]).logits[0]
        got = model.logits(ids, torch.arange(T), torch.tensor([0, T], dtype=torch.int32), T)
    torch.testing.assert_close(got, want, rtol=1e-4, atol=1e-4)
    # two sequences packed into one row = the two sequences run separately
    ids2 = torch.randint(0, cfg.vocab_size, (9,))
    with torch.no_grad():
        packed = model.logits(torch.cat([ids, ids2]), torch.cat([torch.arange(T), torch.arange(9)]),
                              torch.tensor([0, T, T + 9], dtype=torch.int32), T)
        want2 = hf_model(input_ids=ids2[None]).logits[0]
    torch.testing.assert_close(packed[:T], want, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(packed[T:], want2, rtol=1e-4, atol=1e-4)
    # and back: the same tensors under the same names
    back = hf.state_dict_to_hf(model.state_dict(), cfg)
    ref_sd = hf_model.state_dict()
    assert set(back) == set(ref_sd)
    for k in ref_sd:
        assert torch.equal(back[k], ref_sd[k]), k
    # a checkpoint folder written here loads in transformers, and loads here again
    hf.save_hf_checkpoint(str(tmp_path), model.state_dict(), cfg, dtype=torch.float32)
    again = transformers.AutoModelForCausalLM.from_pretrained(str(tmp_path), attn_implementation="eager").float().eval()
    with torch.no_grad():
        torch.testing.assert_close(again(input_ids=ids[None]).logits[0], want, rtol=1e-4, atol=1e-4)
    cfg2, sd2 = hf.load_hf_checkpoint(str(tmp_path))
    assert cfg2 == cfg and set(sd2) == set(sd) and all(torch.equal(sd2[k], sd[k]) for k in sd)
    loaded = hf.decoder_from_hf(str(tmp_path))
    with torch.no_grad():
        torch.testing.assert_close(loaded.logits(ids, torch.arange(T), torch.tensor([0, T], dtype=torch.int32), T), got)


def test_unsupported_hf_configs_are_refused():
    from odc_b200.models import hf
    base = dict(model_type="llama", vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=1,
                num_attention_heads=4, num_key_value_heads=2)
    with pytest.raises(NotImplementedError, match="rotary scaling"):
        hf.config_from_hf(dict(base, rope_scaling={"rope_type": "yarn", "factor": 32.0}))
    with pytest.raises(NotImplementedError, match="model_type"):
        hf.config_from_hf(dict(base, model_type="gpt2"))
    with pytest.raises(NotImplementedError, match="o_proj"):
        hf.config_from_hf(dict(base, attention_bias=True))
    cfg = hf.config_from_hf(dict(base, rope_theta=5e5, activation_checkpointing=None), activation_checkpointing=True)
    assert cfg.rope_theta == 5e5 and cfg.activation_checkpointing and cfg.head_dim == 16


def _train_hf_model(rank, world, mode):
    """The reference's own usage: a Hugging Face causal LM, ``fully_shard`` per decoder layer + root, the patch
    calls in the order its README gives, packed sequences through ``position_ids``; ranks run 2 and 3 microbatches."""
    import torch.distributed as dist
    from torch.distributed.fsdp import fully_shard

    import odc_b200 as odc
    from odc_b200.fsdp import fsdp2

    conf = transformers.Qwen2Config(vocab_size=257, hidden_size=64, intermediate_size=112, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, tie_word_embeddings=False)
    conf._attn_implementation = "eager"
    torch.manual_seed(0)
    model = transformers.Qwen2ForCausalLM(conf).float()
    if mode == "odc":
        odc.init_nvshmem("cpu", 256 << 20)
        fsdp2.patch_fsdp2()
    for layer in model.model.layers:
        fully_shard(layer)
    fully_shard(model)
    if mode == "odc":
        for layer in model.model.layers:
            fsdp2.patch_lazy_init(layer)
        fsdp2.patch_lazy_init(model)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    losses = []
    for step in range(3):
        if mode == "odc":
            fsdp2.pre_minibatch_start(model)
        mine = 2 + rank
        n_micro = mine if mode == "odc" else 2 + world - 1   # lock-step FSDP pads the short rank with zero-weight work
        total = torch.zeros(())
        for i in range(n_micro):
            g = torch.Generator().manual_seed(1000 * step + 10 * (i if i < mine else 0) + rank)
            ids = torch.randint(0, 257, (1, 24), generator=g)
            out = model(input_ids=ids, labels=ids)
            loss = out.loss / 4.0 * (1.0 if i < mine else 0.0)
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


def test_patch_works_on_a_hugging_face_model_as_in_the_reference_readme():
    import sys, os
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from _mp import assert_mostly_close, run_pair
    a, b = run_pair(_train_hf_model, 2)
    assert a[0][0] == pytest.approx(b[0][0], rel=1e-4), (a[0][0], b[0][0])
    for k in a[0][1]:
        assert_mostly_close(a[0][1][k], b[0][1][k], rtol=5e-3, atol=2e-4)


def _train_hf_model_fsdp1(rank, world, mode):
    """The same with FSDP1 flat parameters, in the reference README's order (patch before ``FSDP(...)``)."""
    import torch.distributed as dist
    from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
    from torch.distributed.fsdp.wrap import ModuleWrapPolicy
    from transformers.models.qwen2.modeling_qwen2 import Qwen2DecoderLayer

    import odc_b200 as odc
    from odc_b200.fsdp import fsdp1

    if mode == "odc":
        fsdp1.patch_fsdp1()
        odc.init_nvshmem("cpu", 256 << 20)
    conf = transformers.Qwen2Config(vocab_size=257, hidden_size=64, intermediate_size=112, num_hidden_layers=2,
                                    num_attention_heads=4, num_key_value_heads=2, tie_word_embeddings=False)
    conf._attn_implementation = "eager"
    torch.manual_seed(0)
    model = FSDP(transformers.Qwen2ForCausalLM(conf).float(), auto_wrap_policy=ModuleWrapPolicy({Qwen2DecoderLayer}),
                 device_id=torch.device("cpu"), use_orig_params=False)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    losses = []
    for step in range(3):
        if mode == "odc":
            fsdp1.pre_minibatch_start(model)
        mine = 2 + rank
        n_micro = mine if mode == "odc" else 2 + world - 1
        total = torch.zeros(())
        for i in range(n_micro):
            g = torch.Generator().manual_seed(1000 * step + 10 * (i if i < mine else 0) + rank)
            ids = torch.randint(0, 257, (1, 24), generator=g)
            loss = model(input_ids=ids, labels=ids).loss / 4.0 * (1.0 if i < mine else 0.0)
            loss.backward()
            total += loss.detach()
        if mode == "odc":
            fsdp1.pre_optimizer_step(model)
        opt.step()
        opt.zero_grad()
        dist.all_reduce(total)
        losses.append(float(total))
    with FSDP.summon_full_params(model):
        full = {k: v.detach().clone() for k, v in model.named_parameters()}
    if mode == "odc":
        fsdp1.stop()
    return losses, full


def test_fsdp1_patch_works_on_a_hugging_face_model():
    import sys, os
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from _mp import assert_mostly_close, run_pair
    a, b = run_pair(_train_hf_model_fsdp1, 2)
    assert a[0][0] == pytest.approx(b[0][0], rel=1e-4), (a[0][0], b[0][0])
    for k in a[0][1]:
        assert_mostly_close(a[0][1][k], b[0][1][k], rtol=5e-3, atol=2e-4)


@pytest.mark.parametrize("seed", range(4))
def test_rescaled_rotary_frequencies_match_transformers(seed):
    """``rope_inv_freq`` (llama3 and linear rules) against ``transformers``' own frequency initialisers."""
    import random

    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS

    from odc_b200.ops.reference import rope_inv_freq
    rnd = random.Random(seed)
    head_dim = rnd.choice([32, 64, 128])
    theta = rnd.choice([10000.0, 500000.0, 1000000.0])
    for kind in ("llama3", "linear"):
        params = {"rope_type": kind, "rope_theta": theta, "factor": rnd.choice([2.0, 8.0, 32.0])}
        if kind == "llama3":
            params.update(low_freq_factor=1.0, high_freq_factor=rnd.choice([2.0, 4.0]),
                          original_max_position_embeddings=rnd.choice([64, 2048, 8192]))
        conf = transformers.LlamaConfig(hidden_size=head_dim * 4, num_attention_heads=4, rope_parameters=dict(params))
        want, _ = ROPE_INIT_FUNCTIONS[kind](conf, "cpu")
        got = rope_inv_freq(head_dim, theta, params)
        torch.testing.assert_close(got, want.float(), rtol=1e-6, atol=0)
