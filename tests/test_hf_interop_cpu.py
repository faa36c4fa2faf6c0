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
