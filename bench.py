"""Headline benchmark: training tokens/s on imbalanced variable-length minibatches.

Default workload (--config 3): Llama-3.2-1B-shaped decoder, bf16 compute with fp32 gradient
accumulation, FSDP2 full shard over N GPUs through this package's on-demand engine; each
minibatch is 8 microbatches per rank, each packed up to 16384 tokens from log-normal sequence
lengths (median 512, sigma 1.0, cap 8192) seeded independently per rank.  Synthetic token ids,
random-init weights.  One "step" = one minibatch = forward+backward of every microbatch, the
once-per-minibatch synchronisation and the optimizer step.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference package, if importable
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="odc_b200", choices=["odc_b200", "reference", "stock"])
    ap.add_argument("--config", default="3", choices=["3", "4", "5"],
                    help="workload: 3 = Llama-3.2-1B FSDP2 full shard (headline), 4 = Llama-3-8B HSDP 4x2 + "
                         "reshard_after_forward=4 + activation checkpointing, 5 = Qwen2.5-14B FSDP1 + activation "
                         "checkpointing with long-tail lengths")
    ap.add_argument("--model", default=None)
    ap.add_argument("--microbatches", type=int, default=None)
    ap.add_argument("--token-budget", type=int, default=None)
    ap.add_argument("--uneven", action="store_true", help="ranks run different numbers of microbatches")
    ap.add_argument("--optimizer", default="fused", choices=["fused", "torch"])
    return ap.parse_args()


def reference_arm(args):
    """Run the unmodified reference from baseline/_ref through its own API, or say why not."""
    ref = os.path.join(REPO, "baseline", "_ref")
    line = {"impl": "reference"}
    if not os.path.isdir(os.path.join(ref, "odc")):
        line["unavailable"] = "baseline/_ref/odc missing: the reference was not installed"
        print(json.dumps(line)); return 0
    sys.path.insert(0, ref)
    try:
        import odc  # noqa: F401
    except Exception as e:  # the reference imports nvshmem4py (nvshmem.core) and cuda.core at import time
        line["unavailable"] = (f"reference installed with --no-deps but `import odc` fails: {type(e).__name__}: {e}; "
                               "nvshmem4py / cuda-core are not in the image or the offline wheelhouse")
        print(json.dumps(line)); return 0
    line["unavailable"] = "reference imported but no runner for it is wired up on this image"
    print(json.dumps(line)); return 0


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    import odc_b200 as odc
    from odc_b200 import ops
    from odc_b200.data import LengthSpec, h2d_bytes, make_minibatch, to_device
    from odc_b200.fsdp import fsdp2
    from odc_b200.models import DecoderLM, get_config
    from odc_b200.utils.clocks import ClockSampler

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29512")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)

    use_odc = args.impl == "odc_b200"
    presets = {
        "3": dict(model="llama3.2-1b", microbatches=8, token_budget=16384, engine="fsdp2", hsdp=False, hpz=0, ac=False,
                  spec=LengthSpec("lognormal", lo=16, median=512.0, sigma=1.0, cap=8192),
                  seq="lognormal(median 512, sigma 1.0, cap 8192), packed"),
        "4": dict(model="llama3-8b", microbatches=16, token_budget=32768, engine="fsdp2", hsdp=True, hpz=4, ac=True,
                  spec=LengthSpec("lognormal", lo=16, median=1024.0, sigma=1.2, cap=16384),
                  seq="lognormal(median 1024, sigma 1.2, cap 16384), packed"),
        "5": dict(model="qwen2.5-14b", microbatches=8, token_budget=32768, engine="fsdp1", hsdp=False, hpz=0, ac=True,
                  spec=LengthSpec("longtail", short=(256, 2048), long=(8192, 32768), long_frac=0.25),
                  seq="75% uniform[256,2048] + 25% uniform[8192,32768], packed"),
    }
    wl = presets[args.config]
    args.model = args.model or wl["model"]
    args.microbatches = args.microbatches or wl["microbatches"]
    args.token_budget = args.token_budget or wl["token_budget"]
    cfg = get_config(args.model, activation_checkpointing=wl["ac"])
    torch.manual_seed(0)
    engine = wl["engine"]
    if engine == "fsdp1":
        from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
        from torch.distributed.fsdp import MixedPrecision
        from torch.distributed.fsdp.wrap import ModuleWrapPolicy

        from odc_b200.fsdp import fsdp1
        from odc_b200.models import DecoderLayer
        if use_odc:
            fsdp1.patch_fsdp1(reduce_dtype=torch.float32)
            odc.init_nvshmem(device)
        with torch.device(device):
            model = DecoderLM(cfg)
        model.reset_parameters(seed=0)
        model = FSDP(model, auto_wrap_policy=ModuleWrapPolicy({DecoderLayer}), device_id=device, use_orig_params=False,
                     mixed_precision=MixedPrecision(param_dtype=torch.bfloat16, reduce_dtype=torch.float32,
                                                    buffer_dtype=torch.bfloat16))
        args.optimizer = "torch"
        opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01, fused=True)
        parallelism = f"fsdp1-dp{world}"
    else:
        with torch.device(device):
            model = DecoderLM(cfg)
        model.reset_parameters(seed=0)
        use_hsdp = wl["hsdp"] and world >= 4 and world % 2 == 0
        shard_size = world // 2 if use_hsdp else world
        hpz = wl["hpz"] if (use_odc and wl["hpz"] and shard_size % wl["hpz"] == 0) else 0
        if use_odc:
            odc.init_nvshmem(device)
            fsdp2.patch_fsdp2(enable_hpz=bool(hpz))
        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
        kw = {"mp_policy": mp}
        parallelism = f"fsdp2-dp{world}"
        if use_hsdp:
            from torch.distributed.device_mesh import init_device_mesh
            kw["mesh"] = init_device_mesh("cuda", (2, world // 2), mesh_dim_names=("dp_replicate", "dp_shard"))
            parallelism = f"hsdp-replicate2-shard{world // 2}"
        if hpz:
            kw["reshard_after_forward"] = hpz
            parallelism += f"-hpz{hpz}"
        if wl["ac"]:
            parallelism += "-actckpt"
        for layer in model.layers:
            fully_shard(layer, **kw)
        fully_shard(model, **kw)
        if use_odc:
            for m in list(model.layers) + [model]:
                fsdp2.patch_lazy_init(m)
        if use_odc and args.optimizer == "fused":
            opt = fsdp2.FusedAdamW(model, lr=1e-4, weight_decay=0.01)
        else:
            args.optimizer = "torch"
            opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01, fused=True)

    spec = wl["spec"]
    n_micro = args.microbatches
    if args.uneven:
        n_micro = max(1, args.microbatches - (rank % 3))
    pool = [make_minibatch(rank, s, cfg.vocab_size, spec, n_micro, args.token_budget, seed=1234, pin=True)
            for s in range(2)]
    pool_dev = [[to_device(mb, device) for mb in mbs] for mbs in pool]
    tokens_per_step = [sum(mb["num_tokens"] for mb in mbs) for mbs in pool]

    if use_odc and engine == "fsdp1":
        fsdp1.pre_minibatch_start(model)

    def step(mbs, from_host: bool):
        if use_odc and engine == "fsdp2":
            fsdp2.pre_minibatch_start(model)
        total = None
        for mb in mbs:
            if from_host:
                mb = to_device(mb, device)
            loss = model(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"],
                         labels=mb["labels"], loss_scale=mb["loss_scale"])
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        if use_odc and engine == "fsdp2":
            fsdp2.pre_optimizer_step(model, materialize_grads=(args.optimizer != "fused"))
        elif use_odc:
            fsdp1.pre_optimizer_step(model)
        opt.step()
        opt.zero_grad()
        if use_odc and engine == "fsdp1":
            fsdp1.pre_minibatch_start(model)
        return total

    def timed(from_host: bool, steps: int):
        src = pool if from_host else pool_dev
        dist.barrier(); torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wall0 = time.perf_counter()
        t0.record()
        toks, last = 0, None
        for i in range(steps):
            loss = step(src[i % len(src)], from_host)
            toks += tokens_per_step[i % len(src)]
            if from_host:
                last = float(loss.item())  # device -> host read of the step's result, every step
        t1.record()
        torch.cuda.synchronize(); dist.barrier()
        wall = time.perf_counter() - wall0
        ms = t0.elapsed_time(t1) if not from_host else wall * 1e3
        stat = torch.tensor([ms, float(toks)], dtype=torch.float64, device=device)
        mx = stat.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stat.clone(); dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        return float(mx[0]), float(sm[1]), last

    for i in range(args.warmup):
        step(pool_dev[i % len(pool_dev)], False)
    def comm_launches():
        if not use_odc:
            return 0
        if engine == "fsdp2":
            return fsdp2.transport_launches()
        return sum(getattr(svc.transport, "launches", 0) for svc in (fsdp1.get_gather_service(), fsdp1.get_reduction_service())
                   if svc is not None)

    launches0 = ops.kernel_launches() + comm_launches()
    sampler = ClockSampler(gpu_index=local_rank).start() if rank == 0 else None
    ms, toks, _ = timed(False, args.steps)
    clocks = sampler.stop() if sampler else {}
    launches = ops.kernel_launches() + comm_launches() - launches0
    e2e_ms, e2e_toks, last_loss = timed(True, args.steps)

    if rank == 0:
        value = toks / (ms / 1e3)
        line = {
            "metric": "tokens/s, imbalanced varlen minibatches", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic token ids, random-init weights", "impl": args.impl,
            "config": {"model": args.model, "global_batch": f"{world}x{n_micro} microbatches x <= {args.token_budget} tokens",
                       "seq_len": wl["seq"], "parallelism": parallelism, "workload": f"config {args.config}",
                       "tokens_per_step": toks / args.steps, "l2": "working set (params+activations, >10 GB) exceeds the 126 MB L2",
                       "optimizer": args.optimizer, "gemm": ops.gemm_backend(), "attention": ops.attn_backend(),
                       "params": cfg.num_params()},
            "clocks": {k: clocks.get(k) for k in ("sm_mhz", "sm_max_mhz", "reasons")},
            "e2e": {"value": e2e_toks / (e2e_ms / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": sum(h2d_bytes(mb) for mb in pool[0]), "d2h_bytes_per_step": 4,
                    "timing": "wall clock around pinned-host H2D + step + loss.item(), max over ranks",
                    "last_loss": last_loss},
            "gpu_launches": launches,
        }
        print(json.dumps(line))
    if use_odc and engine == "fsdp2":
        fsdp2.stop()
    elif use_odc:
        fsdp1.stop()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
