"""LLM trainer on FSDP1 (counterpart of the reference's examples/llm_training/torch_fsdp.py).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        examples/llm_training/train_fsdp1.py --model_name qwen2.5-1.5b --activation-checkpointing
"""
import os

import torch
import torch.distributed as dist
from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
from torch.distributed.fsdp import MixedPrecision
from torch.distributed.fsdp.wrap import ModuleWrapPolicy

from args import get_args
from common import (Timer, build_decoder, export_model, init_device, init_logging, log_metrics, log_packing,
                    make_dataset, mark_done, memory_metrics, microbatch_loss, model_config)

import odc_b200 as odc
from odc_b200.data import to_device
from odc_b200.fsdp import fsdp1
from odc_b200.models import DecoderLayer

ODC = os.environ.get("ODC", "1") == "1"
if ODC:
    fsdp1.patch_fsdp1(reduce_dtype=torch.float32)  # before any FSDP(...) is constructed


def main():
    args = get_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = init_device(args, rank)
    if ODC:
        odc.init_nvshmem(dev)
    cfg = model_config(args)
    model = build_decoder(args, cfg, dev)
    mp = MixedPrecision(param_dtype=torch.bfloat16, reduce_dtype=torch.float32, buffer_dtype=torch.bfloat16)
    model = FSDP(model, auto_wrap_policy=ModuleWrapPolicy({DecoderLayer}), device_id=dev, use_orig_params=False,
                 mixed_precision=mp)
    use_fused = ODC and os.environ.get("FUSED_OPTIMIZER", "1") == "1"
    opt = fsdp1.FusedAdamW(model, lr=args.lr, weight_decay=0.01) if use_fused else \
        torch.optim.AdamW(model.parameters(), lr=args.lr, weight_decay=0.01)
    data = make_dataset(args, cfg, rank, world, ODC)
    init_logging(args, rank)
    if ODC:
        fsdp1.pre_minibatch_start(model)
    for step in range(min(args.steps, len(data))):
        times = {}
        microbatches = data[step]
        log_packing(data, rank)
        with Timer("minibatch_time", times):
            total = torch.zeros((), device=dev)
            tokens = 0
            for mb in microbatches:
                mb = to_device(mb, dev)
                tokens += mb["num_tokens"]
                loss = microbatch_loss(args, model, mb)
                if not args.forward_only:
                    loss.backward()
                total += loss.detach()
            if not args.forward_only:
                with Timer("sync_time", times):
                    if ODC:
                        fsdp1.pre_optimizer_step(model, materialize_grads=not use_fused)
                with Timer("optimizer_step_time", times):
                    grad_norm = opt.clip_grad_norm_(1.0) if use_fused else model.clip_grad_norm_(1.0)
                    opt.step()
                    opt.zero_grad()
                if ODC:
                    fsdp1.pre_minibatch_start(model)
        dist.all_reduce(total)
        tok = torch.tensor([tokens], device=dev)
        dist.all_reduce(tok)
        log_metrics(rank, step, {"loss": float(total) / world, "tokens": int(tok), "microbatches": len(microbatches),
                                 "tokens_per_s": int(tok) / times["minibatch_time"], **times, **memory_metrics()})
    export_model(args, model, cfg)
    mark_done(args)
    if ODC:
        fsdp1.stop()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
