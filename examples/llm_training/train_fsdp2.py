"""LLM trainer on FSDP2 (counterpart of the reference's examples/llm_training/torch_fsdp2.py).

Environment switches: ``ODC`` (default 1), ``HPZ``, ``HSDP``, ``ENGINE=fused`` (the fused-kernel decoder engine);
``TORCH_PROFILED=1`` writes a chrome trace per rank; ``CUDA_PROFILED=1`` brackets the last minibatch with
cudaProfilerStart/Stop.

``--checkpoint-dir`` / ``--checkpoint-every``: model + optimizer + next step are saved there and a restarted job
resumes from the newest one.  A peer that left or a bounded wait that ran out ends a rank with exit code 75 and one
JSON line (``ODC_HEARTBEAT_S`` > 0 makes a departed rank visible at the next host barrier instead of after the wait
budget); ``ODC_INJECT_LEAVE="<rank>:<step>"`` rehearses that on the host.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        examples/llm_training/train_fsdp2.py --model_name llama3.2-1b --packing_method DynamicDiffMicro --max_token_len 16384
"""
import os
import time

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import init_device_mesh
from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

from args import get_args
from common import (Timer, build_decoder, export_model, init_device, init_logging, inject_leave, log_metrics, log_packing,
                    make_dataset, mark_done, maybe_save, memory_metrics, microbatch_loss, model_config, open_checkpoint,
                    run_guarded)

import odc_b200 as odc
from odc_b200.data import to_device
from odc_b200.fsdp import fsdp2
from odc_b200.utils.nvtx import nvtx_range

ODC = os.environ.get("ODC", "1") == "1"
# ENGINE=fused: the decoder on the fused gather+GEMM / weight-gradient+scatter kernels instead of the FSDP2 patch
FUSED = os.environ.get("ENGINE", "fsdp2") == "fused"
HPZ = os.environ.get("HPZ", "0") == "1"
HSDP = os.environ.get("HSDP", "0") == "1"


def main():
    args = get_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = init_device(args, rank)
    cfg = model_config(args)
    if FUSED:
        return main_fused(args, cfg, dev, rank, world)
    if ODC:
        odc.init_nvshmem(dev)
        fsdp2.patch_fsdp2(enable_hpz=HPZ)
    model = build_decoder(args, cfg, dev)
    mesh = init_device_mesh(dev.type, (2, world // 2), mesh_dim_names=("dp_replicate", "dp_shard")) if HSDP \
        else init_device_mesh(dev.type, (world,))
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    raf = (world // 2 if not HSDP else max(1, world // 4)) if HPZ else True
    for layer in model.layers:
        fully_shard(layer, mesh=mesh, mp_policy=mp, reshard_after_forward=raf)
    fully_shard(model, mesh=mesh, mp_policy=mp, reshard_after_forward=raf)
    ck = open_checkpoint(args)
    resume = ck is not None and not ck.is_empty()
    if resume:
        ck.load_model(model)   # before the shards move into the symmetric heap (first forward after patch_lazy_init)
    if ODC:
        for m in list(model.layers) + [model]:
            fsdp2.patch_lazy_init(m)
    use_fused = ODC and os.environ.get("FUSED_OPTIMIZER", "1") == "1"
    opt = fsdp2.FusedAdamW(model, lr=args.lr, weight_decay=0.01) if use_fused else \
        torch.optim.AdamW(model.parameters(), lr=args.lr, weight_decay=0.01)
    first_step = 0
    if resume:
        ck.load_optim(model, opt)
        first_step = int(ck.load_meta().get("next_step", 0))
    data = make_dataset(args, cfg, rank, world, ODC)
    init_logging(args, rank)
    prof = None
    if os.environ.get("TORCH_PROFILED", "0") == "1":
        prof = torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA])
        prof.start()
    steps = min(args.steps, len(data))
    for step in range(first_step, steps):
        times = {}
        inject_leave(rank, step)
        if os.environ.get("CUDA_PROFILED", "0") == "1" and step == steps - 1:
            torch.cuda.cudart().cudaProfilerStart()
        microbatches = data[step]
        log_packing(data, rank)
        with Timer("minibatch_time", times):
            if ODC:
                fsdp2.pre_minibatch_start(model)
            t_begin = time.perf_counter()
            total = torch.zeros((), device=dev)
            tokens = 0
            for mb in microbatches:
                with nvtx_range("microbatch"):
                    mb = to_device(mb, dev)
                    tokens += mb["num_tokens"]
                    with torch.set_grad_enabled(not args.forward_only):
                        loss = microbatch_loss(args, model, mb)
                    if not args.forward_only:
                        loss.backward()
                    total += loss.detach()
            with Timer("_drain", times):   # this rank's own work is done here; what follows is waiting for the others
                pass
            times["work_time"] = times.pop("_drain") + (time.perf_counter() - t_begin)
            if not args.forward_only:
                with Timer("sync_time", times):
                    if ODC:
                        fsdp2.pre_optimizer_step(model, materialize_grads=not use_fused)
                with Timer("optimizer_step_time", times):
                    if use_fused:
                        grad_norm = opt.clip_grad_norm_(1.0)
                    else:
                        grad_norm = torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
                    opt.step()
                    opt.zero_grad()
        dist.all_reduce(total)
        tok = torch.tensor([tokens], device=dev)
        dist.all_reduce(tok)
        # share of the minibatch each rank spent NOT working on its own microbatches.  Meaningful with ODC=1, where
        # nothing inside the microbatch loop waits for a peer; under lock-step FSDP the waiting hides inside the
        # collectives of the loop, so the figure reads near zero there and the throughput shows the cost instead.
        work = torch.tensor([times["work_time"]], device=dev, dtype=torch.float64)
        works = [torch.zeros_like(work) for _ in range(world)]
        dist.all_gather(works, work)
        span = max(float(w) for w in works)
        times["idle_share_per_rank"] = [round(1.0 - float(w) / span, 4) for w in works]
        log_metrics(rank, step, {"loss": float(total) / world, "tokens": int(tok), "microbatches": len(microbatches),
                                 "tokens_per_s": int(tok) / times["minibatch_time"],
                                 "grad_norm": float(grad_norm) if not args.forward_only else 0.0, **times, **memory_metrics()})
        maybe_save(args, ck, model, opt, step + 1, last=step == steps - 1)
    if os.environ.get("CUDA_PROFILED", "0") == "1":
        torch.cuda.cudart().cudaProfilerStop()
    if prof is not None:
        prof.stop()
        out_dir = os.environ.get("ODC_OUT_DIR", "bench_out")
        os.makedirs(out_dir, exist_ok=True)
        prof.export_chrome_trace(f"{out_dir}/trace_{args.run_name}_rank{rank}.json")
    export_model(args, model, cfg)
    mark_done(args)
    if ODC:
        fsdp2.stop()
    dist.destroy_process_group()


def main_fused(args, cfg, dev, rank, world):
    """The same loop on ``FusedDecoderLM``: start_minibatch / microbatches / finish_minibatch / optimizer step."""
    from odc_b200.parallel import FusedDecoderLM, FusedOptimizer
    odc.init_nvshmem(dev)
    source = build_decoder(args, cfg, dev) if args.hf_checkpoint else None   # else: the seeded initial weights
    mesh = init_device_mesh(dev.type, (2, world // 2), mesh_dim_names=("dp_replicate", "dp_shard")) if HSDP else None
    model = FusedDecoderLM(cfg, device=dev, seed=0, source=source, mesh=mesh)
    del source
    opt = FusedOptimizer(model, lr=args.lr, weight_decay=0.01)
    ck = open_checkpoint(args)
    first_step = 0
    if ck is not None and not ck.is_empty():
        ck.load_model(model)
        ck.load_optim(model, opt)
        first_step = int(ck.load_meta().get("next_step", 0))
    data = make_dataset(args, cfg, rank, world, True)
    init_logging(args, rank)
    steps = min(args.steps, len(data))
    for step in range(first_step, steps):
        times = {}
        inject_leave(rank, step)
        microbatches = data[step]
        log_packing(data, rank)
        with Timer("minibatch_time", times):
            model.start_minibatch()
            total = torch.zeros((), device=dev)
            tokens = 0
            for mb in microbatches:
                with nvtx_range("microbatch"):
                    mb = to_device(mb, dev)
                    tokens += mb["num_tokens"]
                    with torch.set_grad_enabled(not args.forward_only):
                        loss = model(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"],
                                     labels=mb["labels"], loss_scale=mb["loss_scale"])
                    if not args.forward_only:
                        loss.backward()
                    total += loss.detach()
            grad_norm = 0.0
            if not args.forward_only:
                with Timer("sync_time", times):
                    model.finish_minibatch()
                with Timer("optimizer_step_time", times):
                    grad_norm = float(opt.clip_grad_norm_(1.0))
                    opt.step()
        dist.all_reduce(total)
        tok = torch.tensor([tokens], device=dev)
        dist.all_reduce(tok)
        log_metrics(rank, step, {"loss": float(total) / world, "tokens": int(tok), "microbatches": len(microbatches),
                                 "tokens_per_s": int(tok) / times["minibatch_time"], "grad_norm": grad_norm, **times,
                                 **memory_metrics()})
        maybe_save(args, ck, model, opt, step + 1, last=step == steps - 1)
    export_model(args, model, cfg)
    mark_done(args)
    model.stop()
    dist.destroy_process_group()


if __name__ == "__main__":
    run_guarded(int(os.environ.get("RANK", "0")), main)
