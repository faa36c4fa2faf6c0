"""Hugging Face Llama / Qwen2 checkpoints <-> this package's decoder.

The reference trains ``AutoModelForCausalLM.from_pretrained(...)`` models directly
(examples/llm_training/torch_fsdp2.py:85-106).  This decoder stores the same weights with the
attention and MLP input projections fused (``wqkv = [q | k | v]``, ``w_gate_up = [gate | up]`` along the
output dimension), uses the same rotate-half rotary convention and the same RMSNorm, so a checkpoint
converts by renaming and concatenating; nothing is permuted.

    cfg = config_from_hf(hf_config)
    model = DecoderLM(cfg); model.load_state_dict(state_dict_from_hf(hf_model.state_dict(), cfg))
    # or, for a checkpoint folder on disk (config.json + *.safetensors):
    cfg, sd = load_hf_checkpoint("/path/to/Qwen2.5-1.5B")
    FusedDecoderLM(cfg, source=model)  /  fused_model.load_full_state_dict(sd)  /  Checkpointer

Rotary scaling: ``linear`` and ``llama3`` (Llama 3.1 / 3.2) are carried over as ``DecoderConfig.rope_scaling``; such
models apply the rotation with PyTorch statements, since the rotary kernel derives its frequencies from
``rope_theta`` alone.  Not covered: other rotary scalings (yarn, dynamic, longrope), sliding-window layers, MLP
biases, a bias on ``o_proj``: :func:`config_from_hf` refuses them instead of converting to a model that computes
something else.
"""
from __future__ import annotations

import glob
import json
import os
from typing import Dict, Mapping, Tuple

import torch

from .llama import DecoderConfig

_SUPPORTED = ("llama", "qwen2", "mistral")


def _get(cfg, name, default=None):
    if isinstance(cfg, Mapping):
        return cfg.get(name, default)
    return getattr(cfg, name, default)


def config_from_hf(hf_config, **overrides) -> DecoderConfig:
    """``DecoderConfig`` of a Hugging Face ``LlamaConfig`` / ``Qwen2Config`` / ``MistralConfig`` (object or dict)."""
    kind = _get(hf_config, "model_type", "llama")
    if kind not in _SUPPORTED:
        raise NotImplementedError(f"model_type {kind!r}: supported are {_SUPPORTED}")
    rope = _get(hf_config, "rope_parameters") or _get(hf_config, "rope_scaling") or {}
    rope_type = rope.get("rope_type", rope.get("type", "default")) if isinstance(rope, Mapping) else "default"
    scaling = None
    if rope_type in ("llama3", "linear"):
        keys = ("factor",) if rope_type == "linear" else ("factor", "low_freq_factor", "high_freq_factor",
                                                          "original_max_position_embeddings")
        scaling = {"rope_type": rope_type, **{k: float(rope[k]) for k in keys}}
    elif rope_type not in (None, "default"):
        raise NotImplementedError(f"rotary scaling {rope_type!r} is not implemented (supported: default, linear, llama3)")
    theta = _get(hf_config, "rope_theta")
    if theta is None and isinstance(rope, Mapping):
        theta = rope.get("rope_theta")
    if _get(hf_config, "use_sliding_window", False) or (kind == "mistral" and _get(hf_config, "sliding_window")):
        raise NotImplementedError("sliding-window attention is not implemented")
    if _get(hf_config, "mlp_bias", False):
        raise NotImplementedError("MLP biases are not implemented")
    heads = int(_get(hf_config, "num_attention_heads"))
    hidden = int(_get(hf_config, "hidden_size"))
    head_dim = _get(hf_config, "head_dim") or hidden // heads
    # Qwen2 always has q/k/v biases (and none on o_proj); Llama has them only with attention_bias, and then on o_proj
    # too, which this decoder has no slot for
    qkv_bias = kind == "qwen2"
    if kind != "qwen2" and _get(hf_config, "attention_bias", False):
        raise NotImplementedError("attention_bias=True (a bias on o_proj) is not implemented")
    cfg = DecoderConfig(vocab_size=int(_get(hf_config, "vocab_size")), hidden_size=hidden,
                        intermediate_size=int(_get(hf_config, "intermediate_size")),
                        num_layers=int(_get(hf_config, "num_hidden_layers")), num_heads=heads,
                        num_kv_heads=int(_get(hf_config, "num_key_value_heads") or heads), head_dim=int(head_dim),
                        rms_eps=float(_get(hf_config, "rms_norm_eps", 1e-6)),
                        rope_theta=float(theta if theta is not None else 10000.0),
                        tie_embeddings=bool(_get(hf_config, "tie_word_embeddings", False)), qkv_bias=qkv_bias,
                        init_std=float(_get(hf_config, "initializer_range", 0.02)), rope_scaling=scaling)
    for k, v in overrides.items():
        setattr(cfg, k, v)
    return cfg


def config_to_hf(cfg: DecoderConfig, model_type: str = None) -> Dict:
    """The ``config.json`` fields of the Hugging Face model with this architecture."""
    model_type = model_type or ("qwen2" if cfg.qkv_bias else "llama")
    arch = {"llama": "LlamaForCausalLM", "qwen2": "Qwen2ForCausalLM", "mistral": "MistralForCausalLM"}[model_type]
    extra = {"rope_scaling": dict(cfg.rope_scaling)} if cfg.rope_scaling else {}
    return {**extra, "model_type": model_type, "architectures": [arch], "vocab_size": cfg.vocab_size,
            "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
            "num_hidden_layers": cfg.num_layers, "num_attention_heads": cfg.num_heads,
            "num_key_value_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim, "rms_norm_eps": cfg.rms_eps,
            "rope_theta": cfg.rope_theta, "tie_word_embeddings": cfg.tie_embeddings, "hidden_act": "silu",
            "initializer_range": cfg.init_std}


def state_dict_from_hf(hf_sd: Mapping[str, torch.Tensor], cfg: DecoderConfig) -> Dict[str, torch.Tensor]:
    """Weights under ``DecoderLM``'s names from a ``LlamaForCausalLM`` / ``Qwen2ForCausalLM`` state dict."""
    def get(name):
        for prefix in ("model.", ""):
            if prefix + name in hf_sd:
                return hf_sd[prefix + name]
        raise KeyError(f"{name} not in the checkpoint")

    out = {"embed.weight": get("embed_tokens.weight"), "norm.weight": get("norm.weight")}
    for i in range(cfg.num_layers):
        a, m = f"layers.{i}.self_attn.", f"layers.{i}.mlp."
        out[f"layers.{i}.attn_norm.weight"] = get(f"layers.{i}.input_layernorm.weight")
        out[f"layers.{i}.mlp_norm.weight"] = get(f"layers.{i}.post_attention_layernorm.weight")
        out[f"layers.{i}.attn.wqkv"] = torch.cat([get(a + "q_proj.weight"), get(a + "k_proj.weight"),
                                                  get(a + "v_proj.weight")], dim=0)
        if cfg.qkv_bias:
            out[f"layers.{i}.attn.bqkv"] = torch.cat([get(a + "q_proj.bias"), get(a + "k_proj.bias"),
                                                      get(a + "v_proj.bias")], dim=0)
        out[f"layers.{i}.attn.wo"] = get(a + "o_proj.weight")
        out[f"layers.{i}.mlp.w_gate_up"] = torch.cat([get(m + "gate_proj.weight"), get(m + "up_proj.weight")], dim=0)
        out[f"layers.{i}.mlp.w_down"] = get(m + "down_proj.weight")
    if not cfg.tie_embeddings:
        out["lm_head"] = hf_sd["lm_head.weight"] if "lm_head.weight" in hf_sd else get("embed_tokens.weight").clone()
    want = (cfg.qkv_dim, cfg.hidden_size)
    if tuple(out["layers.0.attn.wqkv"].shape) != want:
        raise ValueError(f"fused QKV weight has shape {tuple(out['layers.0.attn.wqkv'].shape)}, the config says {want}")
    return out


def state_dict_to_hf(sd: Mapping[str, torch.Tensor], cfg: DecoderConfig) -> Dict[str, torch.Tensor]:
    """The inverse of :func:`state_dict_from_hf` (names of ``LlamaForCausalLM`` / ``Qwen2ForCausalLM``)."""
    nq, nkv = cfg.num_heads * cfg.head_dim, cfg.num_kv_heads * cfg.head_dim
    out = {"model.embed_tokens.weight": sd["embed.weight"], "model.norm.weight": sd["norm.weight"]}
    for i in range(cfg.num_layers):
        a, m = f"model.layers.{i}.self_attn.", f"model.layers.{i}.mlp."
        out[f"model.layers.{i}.input_layernorm.weight"] = sd[f"layers.{i}.attn_norm.weight"]
        out[f"model.layers.{i}.post_attention_layernorm.weight"] = sd[f"layers.{i}.mlp_norm.weight"]
        q, k, v = sd[f"layers.{i}.attn.wqkv"].split([nq, nkv, nkv], dim=0)
        out[a + "q_proj.weight"], out[a + "k_proj.weight"], out[a + "v_proj.weight"] = q, k, v
        if cfg.qkv_bias:
            bq, bk, bv = sd[f"layers.{i}.attn.bqkv"].split([nq, nkv, nkv], dim=0)
            out[a + "q_proj.bias"], out[a + "k_proj.bias"], out[a + "v_proj.bias"] = bq, bk, bv
        out[a + "o_proj.weight"] = sd[f"layers.{i}.attn.wo"]
        g, u = sd[f"layers.{i}.mlp.w_gate_up"].split([cfg.intermediate_size, cfg.intermediate_size], dim=0)
        out[m + "gate_proj.weight"], out[m + "up_proj.weight"] = g, u
        out[m + "down_proj.weight"] = sd[f"layers.{i}.mlp.w_down"]
    out["lm_head.weight"] = sd["embed.weight"] if cfg.tie_embeddings else sd["lm_head"]
    return {k: v.contiguous() for k, v in out.items()}


def load_hf_checkpoint(path: str, **config_overrides) -> Tuple[DecoderConfig, Dict[str, torch.Tensor]]:
    """``(config, state dict under DecoderLM's names)`` from a checkpoint folder: ``config.json`` plus
    ``*.safetensors`` shards (or ``pytorch_model*.bin``).  Reads on the CPU; nothing is downloaded."""
    with open(os.path.join(path, "config.json")) as f:
        cfg = config_from_hf(json.load(f), **config_overrides)
    hf_sd: Dict[str, torch.Tensor] = {}
    shards = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if shards:
        from safetensors.torch import load_file
        for s in shards:
            hf_sd.update(load_file(s, device="cpu"))
    else:
        bins = sorted(glob.glob(os.path.join(path, "pytorch_model*.bin")))
        if not bins:
            raise FileNotFoundError(f"no *.safetensors or pytorch_model*.bin under {path}")
        for b in bins:
            hf_sd.update(torch.load(b, map_location="cpu", weights_only=True))
    return cfg, state_dict_from_hf(hf_sd, cfg)


def save_hf_checkpoint(path: str, sd: Mapping[str, torch.Tensor], cfg: DecoderConfig, dtype: torch.dtype = torch.bfloat16,
                       model_type: str = None) -> None:
    """Write ``config.json`` + ``model.safetensors`` that ``AutoModelForCausalLM.from_pretrained(path)`` reads.
    ``sd`` has ``DecoderLM``'s names with whole tensors (``model.state_dict()`` of an unsharded model, or
    ``FusedDecoderLM.full_state_dict()``); call on one rank."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    hf = {k: v.detach().to("cpu", dtype).contiguous() for k, v in state_dict_to_hf(sd, cfg).items()}
    if cfg.tie_embeddings:
        hf.pop("lm_head.weight")   # tied checkpoints store the matrix once
    save_file(hf, os.path.join(path, "model.safetensors"), metadata={"format": "pt"})
    conf = config_to_hf(cfg, model_type)
    conf["torch_dtype"] = str(dtype).replace("torch.", "")
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(conf, f, indent=2)


def decoder_from_hf(path: str, device=None, **config_overrides):
    """An unsharded ``DecoderLM`` (fp32 parameters on ``device``) holding the checkpoint folder's weights: wrap it
    with ``fully_shard`` / ``FSDP(...)``, or hand it to ``FusedDecoderLM(cfg, source=...)``."""
    from .llama import DecoderLM
    cfg, sd = load_hf_checkpoint(path, **config_overrides)
    with torch.device(device or "cpu"):
        model = DecoderLM(cfg)
    model.load_state_dict(sd)
    return model
