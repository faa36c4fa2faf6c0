"""Shared code of the two primitive micro-benchmarks (launched with torch.distributed.run)."""
from __future__ import annotations

import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

NVLINK_GBS = 770.0  # measured peer-copy bandwidth per direction per GPU of an 8 x B200 node (900 nominal)


CPU = os.environ.get("ODC_BENCH_CPU", "0") == "1"  # functional run on CPU ranks (gloo + host-shm heap)


def setup():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if CPU:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        return rank, world, torch.device("cpu")
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    return rank, world, dev


def sync():
    if not CPU:
        torch.cuda.synchronize()


def reduce_scatter_sum(out: torch.Tensor, inp: torch.Tensor) -> None:
    """The library collective the on-demand reduction is compared with (gloo has none: all-reduce, keep my row)."""
    if not CPU:
        dist.reduce_scatter_tensor(out, inp)
        return
    full = inp.clone()
    dist.all_reduce(full)
    out.copy_(full.view(dist.get_world_size(), -1)[dist.get_rank()])


def device_time_ms(fn, iters: int, warmup: int = 3) -> float:
    """Median over iterations of the max-over-ranks device time of ``fn`` (CUDA events; wall clock on CPU ranks)."""
    for _ in range(warmup):
        fn()
    if CPU:
        import time
        ts = []
        for _ in range(iters):
            dist.barrier()
            t0 = time.perf_counter()
            fn()
            t = torch.tensor([(time.perf_counter() - t0) * 1e3])
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts.append(float(t))
        return statistics.median(ts)
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ts.append(float(t))
    return statistics.median(ts)


def sizes_from_argv(default_lo=64 << 10, default_hi=1 << 30):
    lo, hi = default_lo, default_hi
    for a in sys.argv[1:]:
        # names chosen so that torch.distributed.run's own parser does not claim them by prefix
        if a.startswith("--min=") or a.startswith("--size-min="):
            lo = int(a.split("=")[1])
        if a.startswith("--size-max="):
            hi = int(a.split("=")[1])
    out, s = [], lo
    while s <= hi:
        out.append(s)
        s *= 2
    return out


def emit(rank, rows, name):
    if rank != 0:
        return
    out_dir = os.environ.get("ODC_OUT_DIR", "bench_out")
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, name), "w") as f:
        json.dump(rows, f, indent=1)
