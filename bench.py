"""Headline benchmark: training tokens/s on imbalanced variable-length minibatches.

Default workload (--config 3): Llama-3.2-1B-shaped decoder, bf16 compute with fp32 gradient
accumulation, parameters, gradients and optimizer state fully sharded over N GPUs, trained through this
package's on-demand engine (default: the fused-kernel engine, whose linears pull weight shards inside the GEMM
kernel and reduce weight gradients into their owners from the GEMM epilogue after every microbatch;
``--engine fsdp2`` runs the on-demand patch of PyTorch FSDP2 instead); each
minibatch is 8 microbatches per rank, each packed up to 16384 tokens from log-normal sequence
lengths (median 512, sigma 1.0, cap 8192) seeded independently per rank.  Synthetic token ids,
random-init weights.  One "step" = one minibatch = forward+backward of every microbatch, the
once-per-minibatch synchronisation and the optimizer step.

A default run times two arms in the same process, on the same model, seeds and data:
  1. the library baseline: stock PyTorch FSDP2 over NCCL with cuBLAS GEMMs, flash-attn and
     torch's fused AdamW (what the reference's trainer runs with ODC=0,
     examples/llm_training/torch_fsdp2.py:50,179-192), a few timed steps;
  2. this package's engine and kernels, --steps timed steps.
``value`` is arm 2; ``vs_baseline`` is arm 2 / arm 1 (the reference publishes no number).

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference package, if importable
    python bench.py --impl stock ...          # only the stock-FSDP arm (own kernels unless ODC_GEMM/ODC_ATTN say otherwise)
"""
from __future__ import annotations

import argparse
import gc
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
                         "reshard_after_forward=int + activation checkpointing, 5 = Qwen2.5-14B FSDP1 + activation "
                         "checkpointing with long-tail lengths")
    ap.add_argument("--engine", default=None, choices=["fsdp2", "fsdp1", "fused"],
                    help="fsdp2 / fsdp1: the on-demand patch of PyTorch FSDP; fused: the native sharded decoder whose "
                         "linears run the gather+GEMM and weight-gradient+scatter kernels (default: the config's)")
    ap.add_argument("--model", default=None)
    ap.add_argument("--microbatches", type=int, default=None)
    ap.add_argument("--token-budget", type=int, default=None)
    ap.add_argument("--uneven", action="store_true", help="ranks run different numbers of microbatches (headline arm)")
    ap.add_argument("--uneven-steps", type=int, default=None,
                    help="extra timed steps with unequal microbatch counts per rank, reported under 'uneven' "
                         "(default: 3 when more than one GPU, else 0)")
    ap.add_argument("--optimizer", default="fused", choices=["fused", "torch"])
    ap.add_argument("--grad-sync", default="microbatch", choices=["microbatch", "minibatch"],
                    help="microbatch: gradients are pushed to their owners after every microbatch; minibatch: they are "
                         "accumulated unsharded in fp32 and pushed once, during the last microbatch's backward")
    ap.add_argument("--baseline-steps", type=int, default=5, help="timed steps of the in-process stock arm (0: skip it)")
    ap.add_argument("--hpz", type=int, default=None, help="config 4: size of the secondary partition group")
    ap.add_argument("--pool", type=int, default=8, help="distinct synthetic minibatches per rank, cycled")
    ap.add_argument("--no-e2e", action="store_true",
                    help="skip the second, end-to-end timed region (for the large configurations, where every step costs tens "
                         "of seconds); the line then carries no 'e2e' value")
    return ap.parse_args()


# ------------------------------------------------------------------------------------------------------------
# reference arm: the unmodified reference package through its own public API
# ------------------------------------------------------------------------------------------------------------
def reference_arm(args):
    """Run the unmodified reference from baseline/_ref through its own API, or say why not."""
    ref = os.path.join(REPO, "baseline", "_ref")
    line = {"impl": "reference"}
    say = (lambda l: print(json.dumps(l))) if int(os.environ.get("RANK", "0")) == 0 else (lambda l: None)  # one line per job
    if not os.path.isdir(os.path.join(ref, "odc")):
        line["unavailable"] = "baseline/_ref/odc missing: the reference was not installed"
        say(line); return 0
    sys.path.insert(0, ref)
    try:
        import odc  # noqa: F401
        from odc.fsdp import fsdp2 as ref_fsdp2
    except Exception as e:  # the reference imports nvshmem4py (nvshmem.core) and cuda.core at import time
        line["unavailable"] = (f"reference installed with --no-deps but `import odc` fails: {type(e).__name__}: {e}; "
                               "nvshmem4py / cuda-core are not in the image or the offline wheelhouse")
        say(line); return 0
    try:
        return _run_reference(args, odc, ref_fsdp2, line)
    except Exception as e:
        line["unavailable"] = f"reference imported but its training step failed: {type(e).__name__}: {e}"[:400]
        say(line); return 0


def _run_reference(args, odc, ref_fsdp2, line):
    """Config 3 on the reference's stock code path: Hugging Face Llama (random init), flash-attn-2 varlen through
    packed position ids, FSDP2 ``fully_shard`` per decoder layer + root, ``odc.init_nvshmem`` /
    ``patch_fsdp2`` / ``patch_lazy_init`` / ``pre_minibatch_start`` / ``pre_optimizer_step`` as in the
    reference's README and trainer (examples/llm_training/torch_fsdp2.py:162-204, 263-292).  Nothing of this
    package except the synthetic data generator is on that path."""
    import torch
    import torch.distributed as dist
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard
    from transformers import AutoModelForCausalLM, LlamaConfig

    from odc_b200.data import LengthSpec, make_minibatch, to_device
    if args.config != "3":
        line["unavailable"] = "the reference arm is wired for config 3 only"
        print(json.dumps(line)); return 0
    rank, world, local_rank = (int(os.environ.get(k, d)) for k, d in (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1"); os.environ.setdefault("MASTER_PORT", "29512")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    odc.init_nvshmem()
    ref_fsdp2.patch_fsdp2()
    cfg = LlamaConfig(vocab_size=128256, hidden_size=2048, intermediate_size=8192, num_hidden_layers=16,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=64, rms_norm_eps=1e-5, rope_theta=500000.0,
                      tie_word_embeddings=True, max_position_embeddings=16384, attn_implementation="flash_attention_2")
    torch.manual_seed(0)
    with torch.device(device):
        model = AutoModelForCausalLM.from_config(cfg, torch_dtype=torch.float32)
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    for layer in model.model.layers:
        fully_shard(layer, mp_policy=mp)
    fully_shard(model, mp_policy=mp)
    for m in list(model.model.layers) + [model]:
        ref_fsdp2.patch_lazy_init(m)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01)
    spec = LengthSpec("lognormal", lo=16, median=512.0, sigma=1.0, cap=8192)
    pool = [make_minibatch(rank, s, cfg.vocab_size, spec, 8, 16384, seed=1234, pin=True) for s in range(args.pool)]
    tokens = [sum(mb["num_tokens"] for mb in mbs) for mbs in pool]

    def step(mbs):
        ref_fsdp2.pre_minibatch_start(model)
        total = None
        for mb in mbs:
            mb = to_device(mb, device)
            out = model(input_ids=mb["input_ids"][None], position_ids=mb["position_ids"][None], use_cache=False)
            logp = torch.log_softmax(out.logits[0].float(), dim=-1)
            valid = mb["labels"] >= 0
            nll = -logp.gather(1, mb["labels"].clamp_min(0)[:, None])[:, 0]
            loss = (nll * mb["loss_scale"] * valid).sum()
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        ref_fsdp2.pre_optimizer_step(model)
        opt.step(); opt.zero_grad()
        return total

    for i in range(args.warmup):
        step(pool[i % len(pool)])
    dist.barrier(); torch.cuda.synchronize()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(); toks = 0
    for i in range(args.steps):
        float(step(pool[i % len(pool)]).item()); toks += tokens[i % len(pool)]
    t1.record(); torch.cuda.synchronize(); dist.barrier()
    stat = torch.tensor([t0.elapsed_time(t1), float(toks)], dtype=torch.float64, device=device)
    mx = stat.clone(); dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    sm = stat.clone(); dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    if rank == 0:
        v = float(sm[1]) / (float(mx[0]) / 1e3)
        line.update({"metric": "tokens/s, imbalanced varlen minibatches", "value": v, "unit": "tokens/s", "n_gpus": world,
                     "steps": args.steps, "warmup": args.warmup, "ms_per_step": float(mx[0]) / args.steps,
                     "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
                     "data": "synthetic token ids, random-init weights",
                     "config": {"model": "llama3.2-1b (transformers LlamaForCausalLM)", "parallelism": f"fsdp2-dp{world}",
                                "global_batch": f"{world}x8 microbatches x <= 16384 tokens"},
                     "e2e": {"value": v, "unit": "tokens/s", "timing": "inputs copied from pinned host memory and "
                             "the loss read back every step inside the timed region"}})
        print(json.dumps(line))
    ref_fsdp2.stop()
    dist.destroy_process_group()
    return 0


# ------------------------------------------------------------------------------------------------------------
PRESETS = {
    "3": dict(model="llama3.2-1b", microbatches=8, token_budget=16384, engine="fused", hsdp=False, hpz=0, ac=False,
              spec=("lognormal", dict(lo=16, median=512.0, sigma=1.0, cap=8192)),
              seq="lognormal(median 512, sigma 1.0, cap 8192), packed"),
    "4": dict(model="llama3-8b", microbatches=16, token_budget=32768, engine="fsdp2", hsdp=True, hpz=4, ac=True,
              spec=("lognormal", dict(lo=16, median=1024.0, sigma=1.2, cap=16384)),
              seq="lognormal(median 1024, sigma 1.2, cap 16384), packed"),
    "5": dict(model="qwen2.5-14b", microbatches=8, token_budget=32768, engine="fsdp1", hsdp=False, hpz=0, ac=True,
              spec=("longtail", dict(short=(256, 2048), long=(8192, 32768), long_frac=0.25)),
              seq="75% uniform[256,2048] + 25% uniform[8192,32768], packed"),
}


class Arm:
    """One way of training the workload: builds model + optimizer, runs minibatches, cleans up after itself."""

    def __init__(self, impl, engine, args, wl, cfg, device, world, rank):
        import torch
        import torch.distributed as dist  # noqa: F401
        from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

        import odc_b200 as odc
        from odc_b200.fsdp import fsdp2
        from odc_b200.models import DecoderLM
        self.impl, self.engine, self.args, self.device = impl, engine, args, device
        self.use_odc = impl == "odc_b200"
        self.fsdp1 = self.fsdp2 = None
        self.parallelism = ""
        self.optimizer = args.optimizer
        torch.manual_seed(0)
        if engine == "fused":
            from odc_b200.parallel import FusedDecoderLM, FusedOptimizer
            odc.init_nvshmem(device)
            self.model = FusedDecoderLM(cfg, device=device, seed=0)
            self.opt = FusedOptimizer(self.model, lr=1e-4, weight_decay=0.01)
            self.parallelism = f"full-shard-dp{world} (fused gather+GEMM / weight-gradient+scatter engine)"
            self.optimizer = "fused"
        elif engine == "fsdp1":
            from torch.distributed.fsdp import FullyShardedDataParallel as FSDP
            from torch.distributed.fsdp import MixedPrecision
            from torch.distributed.fsdp.wrap import ModuleWrapPolicy

            from odc_b200.fsdp import fsdp1
            from odc_b200.models import DecoderLayer
            self.fsdp1 = fsdp1
            if self.use_odc:
                fsdp1.patch_fsdp1(reduce_dtype=torch.float32)
                odc.init_nvshmem(device)
            with torch.device(device):
                model = DecoderLM(cfg)
            model.reset_parameters(seed=0)
            self.model = FSDP(model, auto_wrap_policy=ModuleWrapPolicy({DecoderLayer}), device_id=device,
                              use_orig_params=False,
                              mixed_precision=MixedPrecision(param_dtype=torch.bfloat16, reduce_dtype=torch.float32,
                                                             buffer_dtype=torch.bfloat16))
            self.optimizer = "torch"
            self.opt = torch.optim.AdamW(self.model.parameters(), lr=1e-4, weight_decay=0.01, fused=True)
            self.parallelism = f"fsdp1-dp{world}"
            if self.use_odc:
                fsdp1.pre_minibatch_start(self.model)
        else:
            self.fsdp2 = fsdp2
            with torch.device(device):
                model = DecoderLM(cfg)
            model.reset_parameters(seed=0)
            use_hsdp = wl["hsdp"] and world >= 4 and world % 2 == 0
            shard_size = world // 2 if use_hsdp else world
            want_hpz = args.hpz if args.hpz is not None else wl["hpz"]
            hpz = want_hpz if (self.use_odc and want_hpz and shard_size % want_hpz == 0) else 0
            if self.use_odc:
                odc.init_nvshmem(device)
                fsdp2.patch_fsdp2(enable_hpz=bool(hpz))
            kw = {"mp_policy": MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)}
            self.parallelism = f"fsdp2-dp{world}"
            if use_hsdp:
                from torch.distributed.device_mesh import init_device_mesh
                kw["mesh"] = init_device_mesh("cuda", (2, world // 2), mesh_dim_names=("dp_replicate", "dp_shard"))
                self.parallelism = f"hsdp-replicate2-shard{world // 2}"
            if hpz:
                kw["reshard_after_forward"] = hpz
                self.parallelism += f"-hpz{hpz}"
            if wl["ac"]:
                self.parallelism += "-actckpt"
            for layer in model.layers:
                fully_shard(layer, **kw)
            fully_shard(model, **kw)
            if self.use_odc:
                for m in list(model.layers) + [model]:
                    fsdp2.patch_lazy_init(m)
            self.model = model
            if self.use_odc and args.optimizer == "fused":
                self.opt = fsdp2.FusedAdamW(model, lr=1e-4, weight_decay=0.01)
            else:
                self.optimizer = "torch"
                self.opt = torch.optim.AdamW(model.parameters(), lr=1e-4, weight_decay=0.01, fused=True)

    def step(self, mbs, from_host):
        from odc_b200.data import to_device
        m, a = self.model, self.args
        if self.engine == "fused":
            m.start_minibatch()
        elif self.use_odc and self.fsdp2 is not None:
            self.fsdp2.pre_minibatch_start(m)
        total = None
        for i, mb in enumerate(mbs):
            if from_host:
                mb = to_device(mb, self.device)
            last = i == len(mbs) - 1
            if a.grad_sync == "minibatch":
                if self.engine == "fused":
                    m.set_requires_gradient_sync(last)
                elif self.fsdp2 is not None:
                    m.set_requires_gradient_sync(last)
            loss = m(mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"],
                     labels=mb["labels"], loss_scale=mb["loss_scale"])
            loss.backward()
            total = loss.detach() if total is None else total + loss.detach()
        if self.engine == "fused":
            m.finish_minibatch()
        elif self.use_odc and self.fsdp2 is not None:
            self.fsdp2.pre_optimizer_step(m, materialize_grads=(self.optimizer != "fused"))
        elif self.use_odc:
            self.fsdp1.pre_optimizer_step(m)
        self.opt.step()
        self.opt.zero_grad()
        if self.use_odc and self.fsdp1 is not None:
            self.fsdp1.pre_minibatch_start(m)
        return total

    def comm_launches(self):
        if self.engine == "fused":
            return self.model.transport_launches()
        if not self.use_odc:
            return 0
        if self.fsdp2 is not None:
            return self.fsdp2.transport_launches()
        return sum(getattr(svc.transport, "launches", 0)
                   for svc in (self.fsdp1.get_gather_service(), self.fsdp1.get_reduction_service()) if svc is not None)

    def close(self):
        import torch
        if self.engine == "fused":
            self.model.stop()
        elif self.use_odc and self.fsdp2 is not None:
            self.fsdp2.stop()
        elif self.use_odc:
            self.fsdp1.stop()
        self.model = self.opt = None
        gc.collect()
        torch.cuda.empty_cache()


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    from odc_b200 import ops
    from odc_b200.data import LengthSpec, h2d_bytes, make_minibatch, to_device
    from odc_b200.models import get_config
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

    wl = PRESETS[args.config]
    args.model = args.model or wl["model"]
    args.microbatches = args.microbatches or wl["microbatches"]
    args.token_budget = args.token_budget or wl["token_budget"]
    engine = args.engine or wl["engine"]
    cfg = get_config(args.model, activation_checkpointing=wl["ac"])
    spec = LengthSpec(wl["spec"][0], **wl["spec"][1])

    def make_pool(n_micro):
        pool = [make_minibatch(rank, s, cfg.vocab_size, spec, n_micro, args.token_budget, seed=1234, pin=True)
                for s in range(max(1, args.pool))]
        return pool, [[to_device(mb, device) for mb in mbs] for mbs in pool], \
            [sum(mb["num_tokens"] for mb in mbs) for mbs in pool]

    n_micro = max(1, args.microbatches - (rank % 3)) if args.uneven else args.microbatches
    pool, pool_dev, tokens_per_step = make_pool(n_micro)

    def timed(arm, src, tokens, steps, from_host):
        dist.barrier(); torch.cuda.synchronize()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wall0 = time.perf_counter()
        t0.record()
        toks, last = 0, None
        for i in range(steps):
            loss = arm.step(src[i % len(src)], from_host)
            toks += tokens[i % len(src)]
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

    # ---- arm 1: the library baseline (stock FSDP over NCCL, cuBLAS, flash-attn, torch AdamW) -------------------
    baseline = baseline_error = None
    if args.impl == "odc_b200" and args.baseline_steps > 0:
        saved = {k: os.environ.get(k) for k in ("ODC_GEMM", "ODC_ATTN")}
        os.environ["ODC_GEMM"], os.environ["ODC_ATTN"] = "cublas", "flash"
        base_args = argparse.Namespace(**{**vars(args), "optimizer": "torch", "grad_sync": "microbatch"})
        stock_engine = "fsdp1" if wl["engine"] == "fsdp1" else "fsdp2"
        arm = None
        try:
            arm = Arm("stock", stock_engine, base_args, wl, cfg, device, world, rank)
            for i in range(min(3, max(1, args.warmup))):
                arm.step(pool_dev[i % len(pool_dev)], False)
            ms, toks, _ = timed(arm, pool_dev, tokens_per_step, args.baseline_steps, False)
            baseline = {"impl": "stock PyTorch FSDP over NCCL (sync every microbatch), cuBLAS GEMMs, flash-attn varlen, "
                                "torch.optim.AdamW(fused=True); same model, seeds and data, same process",
                        "value": toks / (ms / 1e3), "unit": "tokens/s", "ms_per_step": ms / args.baseline_steps,
                        "steps": args.baseline_steps, "parallelism": arm.parallelism}
        except ImportError as e:   # a library of the stock arm is missing: the headline arm does not need it
            baseline_error = f"stock arm not run: {type(e).__name__}: {e}"[:300]
        if arm is not None:
            arm.close()
        del arm
        for k, v in saved.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v

    # ---- arm 2: the headline ---------------------------------------------------------------------------------
    arm = Arm(args.impl, engine, args, wl, cfg, device, world, rank)
    for i in range(args.warmup):
        arm.step(pool_dev[i % len(pool_dev)], False)
    launches0 = ops.kernel_launches() + arm.comm_launches()
    sampler = ClockSampler(gpu_index=local_rank).start() if rank == 0 else None
    ms, toks, _ = timed(arm, pool_dev, tokens_per_step, args.steps, False)
    clocks = sampler.stop() if sampler else {}
    launches = ops.kernel_launches() + arm.comm_launches() - launches0
    e2e_ms = e2e_toks = last_loss = None
    if not args.no_e2e:
        e2e_ms, e2e_toks, last_loss = timed(arm, pool, tokens_per_step, args.steps, True)

    # ---- the capability the engine exists for: ranks run different numbers of microbatches ---------------------
    uneven = None
    uneven_steps = args.uneven_steps if args.uneven_steps is not None else (3 if world > 1 else 0)
    if uneven_steps > 0 and args.impl == "odc_b200" and not args.uneven:
        counts = [max(1, args.microbatches - (r % 3)) for r in range(world)]
        u_pool, u_dev, u_tokens = make_pool(counts[rank])
        arm.step(u_dev[0], False)
        u_ms, u_toks, _ = timed(arm, u_dev, u_tokens, uneven_steps, False)
        uneven = {"value": u_toks / (u_ms / 1e3), "unit": "tokens/s", "ms_per_step": u_ms / uneven_steps,
                  "steps": uneven_steps, "microbatches_per_rank": counts, "tokens_per_step": u_toks / uneven_steps,
                  "note": "lock-step FSDP cannot run this schedule: every rank would have to launch the same "
                          "collectives the same number of times"}

    if rank == 0:
        value = toks / (ms / 1e3)
        line = {
            "metric": "tokens/s, imbalanced varlen minibatches", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / baseline["value"]) if baseline else None, "dtype": "bf16",
            "data": f"synthetic token ids, random-init weights; {len(pool)} distinct minibatches per rank, cycled",
            "impl": args.impl,
            "config": {"model": args.model, "global_batch": f"{world}x{n_micro} microbatches x <= {args.token_budget} tokens",
                       "seq_len": wl["seq"], "parallelism": arm.parallelism, "workload": f"config {args.config}",
                       "engine": engine, "grad_sync": args.grad_sync,
                       "tokens_per_step": toks / args.steps, "l2": "working set (params+activations, >10 GB) exceeds the 126 MB L2",
                       "optimizer": arm.optimizer, "gemm": ops.gemm_backend(), "attention": ops.attn_backend(),
                       "params": cfg.num_params()},
            "clocks": {k: clocks.get(k) for k in ("sm_mhz", "sm_max_mhz", "reasons")},
            "e2e": None if e2e_ms is None else {
                "value": e2e_toks / (e2e_ms / 1e3), "unit": "tokens/s",
                "h2d_bytes_per_step": sum(h2d_bytes(mb) for mb in pool[0]), "d2h_bytes_per_step": 4,
                "timing": "wall clock around pinned-host H2D + step + loss.item(), max over ranks",
                "last_loss": last_loss},
            "gpu_launches": launches,
            "baseline": baseline,
            "vs_baseline_is": "value / baseline.value (in-process stock arm); the reference publishes no number",
        }
        if uneven is not None:
            line["uneven"] = uneven
        if baseline_error is not None:
            line["baseline_error"] = baseline_error
        print(json.dumps(line))
    arm.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
