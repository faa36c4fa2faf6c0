"""Sequence packing and load balancing across ranks and microbatches.

Capabilities of the reference's packing module (examples/llm_training/packing.py): k-way
number partitioning by largest differencing (Karmarkar-Karp), greedy longest-first, pairwise
swap refinement, first-/best-fit-decreasing bin packing, token-budgeted microbatching with or
without the same microbatch count on every rank, cost models (linear, fitted quadratic, FLOPs)
and the named strategies ``None``, ``DynamicSameMicro``, ``DynamicDiffMicro``, ``LocalSort``,
``DebugUneven``.  ``DynamicDiffMicro`` and ``DebugUneven`` produce a different number of
microbatches per rank, which only an on-demand engine can run.
"""
from __future__ import annotations

import heapq
import math
from typing import Callable, List, Optional, Sequence, Tuple

CostFn = Callable[[Sequence[int]], List[float]]

# ---------------------------------------------------------------------------- cost models
FIT_COEFFS = {  # a*s^2 + b*s (+c), s = len/32000 (packing.py:458-472)
    "1.5b": (1.982122, 2.611821, 0.666759),
    "7b": (4.348357, 8.768377, 0.950719),
}


def cost_linear(lengths: Sequence[int]) -> List[float]:
    return [float(x) for x in lengths]


def make_cost_fit(model: str = "7b", with_constant: bool = False) -> CostFn:
    a, b, c = FIT_COEFFS[model]

    def fn(lengths):
        out = []
        for n in lengths:
            s = n / 32000.0
            out.append(a * s * s + b * s + (c if with_constant else 0.0))
        return out

    return fn


def make_cost_flops(linear_params: float, attn_width: float) -> CostFn:
    """Relative FLOPs of a sequence: ``(P/w + len) * len`` with P matmul parameters, w = heads*head_dim."""

    def fn(lengths):
        return [(linear_params / attn_width + n) / 32000.0 * n / 32000.0 for n in lengths]

    return fn


def get_cost_fn(name: str, **kw) -> CostFn:
    if name == "linear":
        return cost_linear
    if name == "fit":
        return make_cost_fit(kw.get("model", "7b"))
    if name == "flops":
        return make_cost_flops(kw["linear_params"], kw["attn_width"])
    raise ValueError(f"unknown cost model {name!r}")


# ---------------------------------------------------------------------------- partitioning
def greedy_partition(costs: Sequence[float], k: int, equal_size: bool = False) -> List[List[int]]:
    """Longest-processing-time first: heaviest item to the lightest bin."""
    n = len(costs)
    cap = math.ceil(n / k) if equal_size else n
    bins: List[List[int]] = [[] for _ in range(k)]
    loads = [0.0] * k
    for i in sorted(range(n), key=lambda i: (-costs[i], i)):
        j = min((b for b in range(k) if len(bins[b]) < cap), key=lambda b: (loads[b], b))
        bins[j].append(i)
        loads[j] += costs[i]
    return bins


def karmarkar_karp(costs: Sequence[float], k: int, equal_size: bool = False) -> List[List[int]]:
    """k-way largest differencing method.

    A state is k bins sorted by load; two states merge by pairing the heaviest bin of one with
    the lightest of the other.  With ``equal_size`` items are first grouped k at a time (sorted
    by cost) so every bin receives the same count (requires ``len(costs) % k == 0``).
    """
    n = len(costs)
    if equal_size and n % k != 0:
        raise ValueError(f"{n} items cannot be split into {k} equal-sized parts")
    order = sorted(range(n), key=lambda i: (costs[i], i))
    heap: List[Tuple[float, int, List[Tuple[float, List[int]]]]] = []
    uid = 0

    def push(state):
        nonlocal uid
        spread = state[-1][0] - state[0][0]
        heapq.heappush(heap, (-spread, uid, state))
        uid += 1

    if equal_size:
        for g in range(0, n, k):
            grp = order[g:g + k]
            push(sorted(((costs[i], [i]) for i in grp), key=lambda t: t[0]))
    else:
        for i in order:
            push([(0.0, [])] * (k - 1) + [(costs[i], [i])])
    if not heap:
        return [[] for _ in range(k)]
    while len(heap) > 1:
        _, _, a = heapq.heappop(heap)
        _, _, b = heapq.heappop(heap)
        merged = [(a[j][0] + b[k - 1 - j][0], a[j][1] + b[k - 1 - j][1]) for j in range(k)]
        merged.sort(key=lambda t: t[0])
        push(merged)
    final = heap[0][2]
    return [sorted(items) for _, items in final]


def refine_by_swaps(costs: Sequence[float], parts: List[List[int]], max_rounds: int = 100) -> List[List[int]]:
    """Pairwise swaps (or moves) between the heaviest and lightest part while the spread shrinks."""
    parts = [list(p) for p in parts]
    for _ in range(max_rounds):
        loads = [sum(costs[i] for i in p) for p in parts]
        hi = max(range(len(parts)), key=lambda j: loads[j])
        lo = min(range(len(parts)), key=lambda j: loads[j])
        gap = loads[hi] - loads[lo]
        if gap <= 0:
            break
        best, best_gain = None, 0.0
        for x in parts[hi]:
            for y in parts[lo]:
                d = costs[x] - costs[y]
                if 0 < d < gap and (gain := min(d, gap - d)) > best_gain:
                    best, best_gain = (x, y), gain
        if best is None:
            break
        x, y = best
        parts[hi].remove(x); parts[lo].remove(y)
        parts[hi].append(y); parts[lo].append(x)
    return [sorted(p) for p in parts]


def balanced_partitions(lengths: Sequence[int], k: int, equal_size: bool = False,
                        cost_fn: Optional[CostFn] = None, refine: bool = True) -> List[List[int]]:
    costs = (cost_fn or cost_linear)(lengths)
    parts = karmarkar_karp(costs, k, equal_size)
    if refine:
        parts = refine_by_swaps(costs, parts)
    return parts


# ---------------------------------------------------------------------------- bin packing
def bin_pack_decreasing(capacity: int, lengths: Sequence[int], best_fit: bool = True) -> List[List[int]]:
    """First-fit / best-fit decreasing; returns item indices per bin."""
    bins: List[List[int]] = []
    room: List[int] = []
    for i in sorted(range(len(lengths)), key=lambda i: (-lengths[i], i)):
        n = lengths[i]
        if n > capacity:
            raise ValueError(f"sequence of {n} tokens exceeds the budget of {capacity}")
        fits = [b for b in range(len(bins)) if room[b] >= n]
        if fits:
            b = min(fits, key=lambda b: (room[b], b)) if best_fit else fits[0]
            bins[b].append(i); room[b] -= n
        else:
            bins.append([i]); room.append(capacity - n)
    return bins


# ---------------------------------------------------------------------------- microbatching
def rearrange_micro_batches(lengths: Sequence[int], max_token_len: int, same_num_in_dp: bool = False,
                            dp_group=None, sort_by_workload: bool = True,
                            cost_fn: Optional[CostFn] = None) -> List[List[int]]:
    """Split one rank's sequences into cost-balanced microbatches of at most ``max_token_len`` tokens.

    With ``same_num_in_dp`` the microbatch count is raised to the maximum over the data-parallel
    group (what lock-step FSDP needs); otherwise each rank uses only as many as it needs.
    """
    cost_fn = cost_fn or cost_linear
    if not lengths:
        return []
    num = min(len(lengths), max(1, math.ceil(sum(lengths) / max_token_len)))

    def agree(x: int) -> int:
        if not same_num_in_dp:
            return x
        import torch
        import torch.distributed as dist
        if not dist.is_initialized():
            return x
        t = torch.tensor([x], dtype=torch.int64)
        if dist.get_backend(dp_group) == "nccl":
            t = t.cuda()
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=dp_group)
        return int(t.item())

    num = agree(num)
    while True:
        num = min(num, len(lengths)) if not same_num_in_dp else num
        parts = balanced_partitions(lengths, num, equal_size=False, cost_fn=cost_fn) if num <= len(lengths) \
            else balanced_partitions(lengths, len(lengths), cost_fn=cost_fn) + [[] for _ in range(num - len(lengths))]
        over = any(sum(lengths[i] for i in p) > max_token_len for p in parts)
        want = agree(num + 1 if over else num)
        if want == num:
            break
        num = want
    if sort_by_workload:
        parts.sort(key=lambda p: (-sum(cost_fn([lengths[i] for i in p])), min(p) if p else 0))
    return parts


# ---------------------------------------------------------------------------- strategies
def pack_none(lengths, rank, world):
    return [[i] for i in range(rank, len(lengths), world)]


def pack_local_sort(lengths, rank, world):
    return [[i] for i in sorted(range(rank, len(lengths), world), key=lambda i: lengths[i])]


def pack_debug_uneven(lengths, rank, world):
    mine = list(range(rank, len(lengths), world))
    step = 1 if rank % 2 == 0 else 2
    return [mine[i:i + step] for i in range(0, len(mine), step)]


def pack_dynamic(lengths, rank, world, max_token_len, same_micro_num=False, use_bin_packing=False,
                 cost_fn: Optional[CostFn] = None, dp_group=None):
    if max(lengths) > max_token_len:
        raise ValueError(f"longest sequence {max(lengths)} exceeds the token budget {max_token_len}")
    cost_fn = cost_fn or cost_linear
    minis = balanced_partitions(lengths, world, equal_size=same_micro_num, cost_fn=cost_fn)
    mine = minis[rank]
    local_len = [lengths[i] for i in mine]
    if not same_micro_num and use_bin_packing:
        micro = bin_pack_decreasing(max_token_len, local_len, best_fit=True)
    else:
        micro = rearrange_micro_batches(local_len, max_token_len, same_num_in_dp=same_micro_num,
                                        dp_group=dp_group, cost_fn=cost_fn)
    return [[mine[j] for j in mb] for mb in micro]


STRATEGIES_NEEDING_ODC = {"DynamicDiffMicro", "DebugUneven"}


def get_packing_function(method: str, max_token_len: int = 65536, cost_fn: Optional[CostFn] = None,
                         odc_enabled: bool = True, **kw):
    if method in STRATEGIES_NEEDING_ODC and not odc_enabled:
        raise ValueError(f"packing method {method} gives ranks different microbatch counts and needs ODC")
    if method == "None":
        return pack_none
    if method == "LocalSort":
        return pack_local_sort
    if method == "DebugUneven":
        return pack_debug_uneven
    if method in ("DynamicSameMicro", "DynamicDiffMicro"):
        same = method == "DynamicSameMicro"
        return lambda lengths, rank, world: pack_dynamic(lengths, rank, world, max_token_len, same_micro_num=same,
                                                         cost_fn=cost_fn, **kw)
    raise ValueError(f"unknown packing method {method!r}")


def imbalance_report(lengths: Sequence[int], world: int, max_token_len: int,
                     cost_fn: Optional[CostFn] = None) -> dict:
    """Compare lock-step microbatching with per-rank microbatching on one global batch (no process group).

    Lock-step cost of a minibatch is ``sum over microbatch slots of max over ranks``; on-demand cost is
    ``max over ranks of the rank's total``.
    """
    cost_fn = cost_fn or cost_linear

    def per_rank(method_same: bool):
        minis = balanced_partitions(lengths, world, equal_size=method_same, cost_fn=cost_fn)
        out = []
        for mine in minis:
            ll = [lengths[i] for i in mine]
            micro = rearrange_micro_batches(ll, max_token_len, cost_fn=cost_fn)
            out.append([sum(cost_fn([ll[j] for j in mb])) for mb in micro])
        return out

    same = per_rank(True) if len(lengths) % world == 0 else per_rank(False)
    slots = max(len(r) for r in same)
    lockstep = sum(max((r[s] if s < len(r) else 0.0) for r in same) for s in range(slots))
    diff = per_rank(False)
    ondemand = max(sum(r) for r in diff)
    ideal = sum(cost_fn(lengths)) / world
    return {"lockstep_cost": lockstep, "ondemand_cost": ondemand, "ideal_cost": ideal,
            "lockstep_bubble": lockstep / ideal - 1.0, "ondemand_bubble": ondemand / ideal - 1.0,
            "microbatches_lockstep": [len(r) for r in same], "microbatches_ondemand": [len(r) for r in diff]}


def report_main(argv=None) -> None:
    """``python -m odc_b200.data``: predicted idle share of lock-step vs per-rank microbatching."""
    import argparse
    import json

    import numpy as np

    from .synthetic import LengthSpec, sample_lengths
    ap = argparse.ArgumentParser(description=report_main.__doc__)
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--sequences", type=int, default=256, help="sequences in one global minibatch")
    ap.add_argument("--max-token-len", type=int, default=16384)
    ap.add_argument("--dist", default="lognormal", choices=["lognormal", "longtail", "uniform"])
    ap.add_argument("--median", type=float, default=512.0)
    ap.add_argument("--sigma", type=float, default=1.0)
    ap.add_argument("--cap", type=int, default=8192)
    ap.add_argument("--cost-model", default="linear", choices=["linear", "fit"])
    ap.add_argument("--minibatches", type=int, default=20)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    spec = {"lognormal": LengthSpec("lognormal", lo=16, median=a.median, sigma=a.sigma, cap=min(a.cap, a.max_token_len)),
            "longtail": LengthSpec("longtail", long=(a.cap // 2, min(a.cap, a.max_token_len))),
            "uniform": LengthSpec("uniform", lo=16, hi=min(a.cap, a.max_token_len))}[a.dist]
    rng = np.random.default_rng(a.seed)
    cost = get_cost_fn(a.cost_model)
    lock, ond = [], []
    for _ in range(a.minibatches):
        r = imbalance_report(sample_lengths(spec, a.sequences, rng), a.world, a.max_token_len, cost)
        lock.append(r["lockstep_bubble"])
        ond.append(r["ondemand_bubble"])
    print(json.dumps({"world": a.world, "sequences": a.sequences, "dist": a.dist, "minibatches": a.minibatches,
                      "lockstep_idle_share_mean": float(np.mean(lock)), "ondemand_idle_share_mean": float(np.mean(ond)),
                      "lockstep_idle_share_max": float(np.max(lock)), "ondemand_idle_share_max": float(np.max(ond))}))
