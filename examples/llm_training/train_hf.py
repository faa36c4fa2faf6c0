"""The reference's own training recipe on a Hugging Face model class, with this package underneath.

The reference trains ``AutoModelForCausalLM`` (Qwen2 by default) wrapped with ``fully_shard``, flash-attn-2 on packed
rows (``position_ids`` restart at every sequence) and a chunked LM head that returns per-token log-probabilities
(examples/llm_training/torch_fsdp2.py:70-106, 162-204, 263-292).  This script is that recipe: the model class stays
Hugging Face's, the FSDP2 patch of this package replaces the all-gather / reduce-scatter, and the head is
``ops.linear_token_logprobs``.  To run the decoder on this package's own kernels instead, convert the checkpoint
(``--hf-checkpoint`` of ``train_fsdp2.py``).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        examples/llm_training/train_hf.py --hf-checkpoint /path/to/Qwen2.5-1.5B --max_token_len 16384

``ODC=0`` trains the same model with stock FSDP (lock-step microbatch counts: use ``DynamicSameMicro``);
``FSDP1=1`` wraps with ``FullyShardedDataParallel`` flat parameters instead of ``fully_shard`` (the reference's
examples/llm_training/torch_fsdp.py).
On GPUs the attention implementation is ``flash_attention_2`` (the library the reference uses); ``--cpu`` uses eager
attention with an explicit block-diagonal causal mask.
"""
import os

import torch
import torch.distributed as dist
import torch.nn as nn
from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

from args import get_args
from common import Timer, init_device, init_logging, log_metrics, log_packing, make_dataset, mark_done, memory_metrics

import odc_b200 as odc
from odc_b200 import ops
from odc_b200.data import to_device
from odc_b200.fsdp import fsdp1, fsdp2
from odc_b200.models.hf import config_from_hf

ODC = os.environ.get("ODC", "1") == "1"
FSDP1 = os.environ.get("FSDP1", "0") == "1"
if ODC and FSDP1:
    fsdp1.patch_fsdp1(reduce_dtype=torch.float32)   # before any FSDP(...) is constructed


def block_causal_mask(cu_seqlens: torch.Tensor, T: int, dtype: torch.dtype) -> torch.Tensor:
    """Additive ``[1, 1, T, T]`` mask: a token sees the earlier tokens of its own sequence only."""
    seg = torch.bucketize(torch.arange(T, device=cu_seqlens.device), cu_seqlens[1:].long(), right=True)
    idx = torch.arange(T, device=cu_seqlens.device)
    allowed = (seg[:, None] == seg[None, :]) & (idx[:, None] >= idx[None, :])
    return torch.zeros(T, T, dtype=dtype, device=cu_seqlens.device).masked_fill(~allowed, float("-inf"))[None, None]


class PackedCausalLM(nn.Module):
    """Root module: the Hugging Face decoder stack on one packed row, then the chunked log-probability head on the
    (unsharded, because this is the root's forward) LM-head matrix."""

    def __init__(self, hf_model, flash: bool):
        super().__init__()
        self.hf, self.flash = hf_model, flash

    def forward(self, input_ids, position_ids, cu_seqlens, max_seqlen, labels, loss_scale):
        kw = {}
        if not self.flash:
            dtype = self.hf.lm_head.weight.dtype
            kw["attention_mask"] = block_causal_mask(cu_seqlens, input_ids.shape[0], dtype)
        h = self.hf.model(input_ids=input_ids[None], position_ids=position_ids[None], use_cache=False, **kw)
        logp = ops.linear_token_logprobs(h.last_hidden_state[0], self.hf.lm_head.weight, labels)
        return -(logp * loss_scale.float()).sum()


def main():
    import transformers
    args = get_args()
    if not args.hf_checkpoint:
        raise SystemExit("train_hf.py needs --hf-checkpoint <folder with config.json and weights>")
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = init_device(args, rank)
    if ODC:
        odc.init_nvshmem(dev)
        if not FSDP1:
            fsdp2.patch_fsdp2()
    engine = fsdp1 if FSDP1 else fsdp2
    flash = dev.type == "cuda"
    hf = transformers.AutoModelForCausalLM.from_pretrained(
        args.hf_checkpoint, attn_implementation="flash_attention_2" if flash else "eager",
        torch_dtype=torch.float32).to(dev)
    if args.activation_checkpointing:
        hf.gradient_checkpointing_enable()
    cfg = config_from_hf(hf.config)          # only for the dataset's vocabulary size and the cost model
    model = PackedCausalLM(hf, flash)
    if FSDP1:
        from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
        from torch.distributed.fsdp import MixedPrecision
        from torch.distributed.fsdp.wrap import ModuleWrapPolicy
        mp1 = MixedPrecision(param_dtype=torch.bfloat16, reduce_dtype=torch.float32, buffer_dtype=torch.bfloat16)
        model = FSDP(model, auto_wrap_policy=ModuleWrapPolicy({type(hf.model.layers[0])}), device_id=dev,
                     use_orig_params=False, mixed_precision=mp1)
    else:
        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)   # as the reference's trainer
        for layer in hf.model.layers:
            fully_shard(layer, mp_policy=mp)
        fully_shard(model, mp_policy=mp)
        if ODC:
            for m in list(hf.model.layers) + [model]:
                fsdp2.patch_lazy_init(m)
    opt = torch.optim.AdamW(model.parameters(), lr=args.lr, weight_decay=0.01)
    data = make_dataset(args, cfg, rank, world, ODC)
    init_logging(args, rank)
    for step in range(min(args.steps, len(data))):
        times = {}
        microbatches = data[step]
        log_packing(data, rank)
        with Timer("minibatch_time", times):
            if ODC:
                engine.pre_minibatch_start(model)
            total = torch.zeros((), device=dev)
            tokens = 0
            for mb in microbatches:
                mb = to_device(mb, dev)
                tokens += mb["num_tokens"]
                loss = model(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"], mb["labels"],
                             mb["loss_scale"])
                if not args.forward_only:
                    loss.backward()
                total += loss.detach()
            if not args.forward_only:
                with Timer("sync_time", times):
                    if ODC:
                        engine.pre_optimizer_step(model)
                with Timer("optimizer_step_time", times):
                    grad_norm = model.clip_grad_norm_(1.0) if FSDP1 else torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
                    opt.step()
                    opt.zero_grad()
        dist.all_reduce(total)
        tok = torch.tensor([tokens], device=dev)
        dist.all_reduce(tok)
        log_metrics(rank, step, {"loss": float(total) / world, "tokens": int(tok), "microbatches": len(microbatches),
                                 "tokens_per_s": int(tok) / times["minibatch_time"],
                                 "grad_norm": float(grad_norm) if not args.forward_only else 0.0, **times, **memory_metrics()})
    mark_done(args)
    if ODC:
        engine.stop()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
