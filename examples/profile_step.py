"""Kernel-time breakdown of one training step (torch.profiler; shares, not absolutes).

    python examples/profile_step.py [--model llama3.2-1b] [--microbatches 2] [--token-budget 16384]

Prints the top CUDA kernels of one minibatch (forward + backward of every microbatch, the
per-minibatch synchronisation and the optimizer step) by total device time.
"""
from __future__ import annotations

import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="llama3.2-1b")
    ap.add_argument("--microbatches", type=int, default=2)
    ap.add_argument("--token-budget", type=int, default=16384)
    ap.add_argument("--top", type=int, default=25)
    ap.add_argument("--engine", default="fsdp2", choices=["fsdp2", "fused"])
    ap.add_argument("--copies", action="store_true",
                    help="also list the copy / cast operators by input shape and Python call site")
    args = ap.parse_args()
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    import odc_b200 as odc
    from odc_b200.data import LengthSpec, make_minibatch, to_device
    from odc_b200.fsdp import fsdp2
    from odc_b200.models import DecoderLM, get_config

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29577")
    dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    cfg = get_config(args.model)
    odc.init_nvshmem(dev)
    if args.engine == "fused":
        from odc_b200.parallel import FusedDecoderLM, FusedOptimizer
        model = FusedDecoderLM(cfg, device=dev, seed=0)
        opt = FusedOptimizer(model, lr=1e-4)
    else:
        with torch.device(dev):
            model = DecoderLM(cfg)
        model.reset_parameters(seed=0)
        fsdp2.patch_fsdp2()
        mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
        for layer in model.layers:
            fully_shard(layer, mp_policy=mp)
        fully_shard(model, mp_policy=mp)
        for m in list(model.layers) + [model]:
            fsdp2.patch_lazy_init(m)
        opt = fsdp2.FusedAdamW(model, lr=1e-4)
    spec = LengthSpec("lognormal", lo=16, median=512.0, sigma=1.0, cap=8192)
    mbs = [to_device(mb, dev) for mb in make_minibatch(0, 0, cfg.vocab_size, spec, args.microbatches, args.token_budget)]

    def step():
        model.start_minibatch() if args.engine == "fused" else fsdp2.pre_minibatch_start(model)
        for mb in mbs:
            loss = model(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"], labels=mb["labels"],
                         loss_scale=mb["loss_scale"])
            loss.backward()
        model.finish_minibatch() if args.engine == "fused" else fsdp2.pre_optimizer_step(model, materialize_grads=False)
        opt.step()
        opt.zero_grad()

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    with torch.profiler.profile(activities=[torch.profiler.ProfilerActivity.CUDA, torch.profiler.ProfilerActivity.CPU],
                                record_shapes=args.copies, with_stack=args.copies) as prof:
        step()
        torch.cuda.synchronize()
    agg = {}
    for e in prof.events():
        if e.device_type == torch.autograd.DeviceType.CUDA:  # device-side kernels and memcpys only
            t, n = agg.get(e.name, (0.0, 0))
            agg[e.name] = (t + e.device_time, n + 1)
    rows = [(k, t, n) for k, (t, n) in agg.items()]
    rows.sort(key=lambda r: -r[1])
    total = sum(r[1] for r in rows)
    print(f"total device time {total / 1e3:.1f} ms over {sum(r[2] for r in rows)} launches; tokens {sum(mb['num_tokens'] for mb in mbs)}")
    for name, t, n in rows[: args.top]:
        print(f"{t / 1e3:9.2f} ms {100 * t / total:5.1f}%  x{n:<5d} {name[:110]}")
    if args.copies:
        print("\ncopy / cast operators by input shape and call site (count, device ms):")
        groups = {}
        for e in prof.events():
            if e.device_type == torch.autograd.DeviceType.CPU and e.name in ("aten::copy_", "aten::_to_copy", "aten::clone",
                                                                             "aten::contiguous", "aten::add_", "aten::add"):
                site = next((f for f in (e.stack or []) if "odc_b200" in f or "examples" in f), (e.stack or ["?"])[0])
                k = (e.name, str(e.input_shapes)[:60], site[-90:])
                t, n = groups.get(k, (0.0, 0))
                groups[k] = (t + e.device_time_total, n + 1)
        for (name, shapes, site), (t, n) in sorted(groups.items(), key=lambda kv: -kv[1][0])[:40]:
            print(f"x{n:<4d} {t / 1e3:8.2f} ms  {name:16s} {shapes:60s} {site}")
    model.stop() if args.engine == "fused" else fsdp2.stop()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
