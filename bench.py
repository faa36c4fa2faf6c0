"""Headline benchmark: training tokens/s on imbalanced variable-length minibatches.

Workload (BASELINE.json config 3): Llama-3.2-1B-shaped decoder, bf16 compute with fp32 gradient
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
    ap.add_argument("--model", default="llama3.2-1b")
    ap.add_argument("--microbatches", type=int, default=8)
    ap.add_argument("--token-budget", type=int, default=16384)
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
    cfg = get_config(args.model)
    torch.manual_seed(0)
    with torch.device(device):
        model = DecoderLM(cfg)
    model.reset_parameters(seed=0)
    if use_odc:
        odc.init_nvshmem(device)
        fsdp2.patch_fsdp2()
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    for layer in model.layers:
        fully_shard(layer, mp_policy=mp)
    fully_shard(model, mp_policy=mp)
    if use_odc:
        for m in list(model.layers) + [model]:
            fsdp2.patch_lazy_init(m)
    if use_odc and args.optimizer == "fused":
        opt = fsdp2.FusedAdamW(model, lr=1e-4, weight_decay=0.01)
    else:
        opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01, fused=True)

    spec = LengthSpec("lognormal", lo=16, median=512.0, sigma=1.0, cap=8192)
    n_micro = args.microbatches
    if args.uneven:
        n_micro = max(1, args.microbatches - (rank % 3))
    pool = [make_minibatch(rank, s, cfg.vocab_size, spec, n_micro, args.token_budget, seed=1234, pin=True)
            for s in range(2)]
    pool_dev = [[to_device(mb, device) for mb in mbs] for mbs in pool]
    tokens_per_step = [sum(mb["num_tokens"] for mb in mbs) for mbs in pool]

    def step(mbs, from_host: bool):
        if use_odc:
            fsdp2.pre_minibatch_start(model)
        total = None
        for mb in mbs:
            if from_host:
                mb = to_device(mb, device)
            loss = model(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"],
                         labels=mb["labels"], loss_scale=mb["loss_scale"])
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        if use_odc:
            fsdp2.pre_optimizer_step(model)
        opt.step()
        opt.zero_grad()
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
    launches0 = ops.kernel_launches() + (fsdp2.transport_launches() if use_odc else 0)
    sampler = ClockSampler(gpu_index=local_rank).start() if rank == 0 else None
    ms, toks, _ = timed(False, args.steps)
    clocks = sampler.stop() if sampler else {}
    launches = ops.kernel_launches() + (fsdp2.transport_launches() if use_odc else 0) - launches0
    e2e_ms, e2e_toks, last_loss = timed(True, args.steps)

    if rank == 0:
        value = toks / (ms / 1e3)
        line = {
            "metric": "tokens/s, imbalanced varlen minibatches", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic token ids, random-init weights", "impl": args.impl,
            "config": {"model": args.model, "global_batch": f"{world}x{n_micro} microbatches x <= {args.token_budget} tokens",
                       "seq_len": "lognormal(median 512, sigma 1.0, cap 8192), packed", "parallelism": f"fsdp2-dp{world}",
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
    if use_odc:
        fsdp2.stop()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
