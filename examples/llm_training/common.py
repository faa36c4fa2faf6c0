"""Pieces shared by the FSDP1 and FSDP2 trainers."""
import json
import os
import sys
import time

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from odc_b200.data import BatchedDataset, LengthSpec, get_cost_fn, sample_lengths  # noqa: E402


class Timer:
    """Wall-clock timer that synchronises the device on both sides."""

    def __init__(self, name, sink):
        self.name, self.sink = name, sink

    def __enter__(self):
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self.t0 = time.perf_counter()

    def __exit__(self, *exc):
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        self.sink[self.name] = self.sink.get(self.name, 0.0) + time.perf_counter() - self.t0


def init_device(args, rank):
    """Process group + device of this rank: one GPU over NCCL, or (``--cpu``) a CPU rank over gloo."""
    import torch.distributed as dist
    if args.cpu:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
        torch.set_num_threads(max(1, (os.cpu_count() or 2) // int(os.environ.get("WORLD_SIZE", "1"))))
        return dev
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=dev)
    return dev


def model_config(args):
    """The decoder configuration: a preset name, or (``--hf-checkpoint``) the one of a Hugging Face Llama / Qwen2
    checkpoint folder, the way the reference's trainers start from ``from_pretrained`` weights."""
    from odc_b200.models import get_config
    if args.hf_checkpoint:
        import json
        from odc_b200.models.hf import config_from_hf
        with open(os.path.join(args.hf_checkpoint, "config.json")) as f:
            return config_from_hf(json.load(f), activation_checkpointing=args.activation_checkpointing)
    return get_config(args.model_name, activation_checkpointing=args.activation_checkpointing)


def build_decoder(args, cfg, dev):
    """An unsharded ``DecoderLM`` on ``dev`` with the run's initial weights (seeded, or the checkpoint's)."""
    from odc_b200.models import DecoderLM
    with torch.device(dev):
        model = DecoderLM(cfg)
    if args.hf_checkpoint:
        from odc_b200.models.hf import load_hf_checkpoint
        _, sd = load_hf_checkpoint(args.hf_checkpoint)
        model.load_state_dict(sd)   # copies into the parameters on ``dev``, keeps their fp32 dtype
    else:
        model.reset_parameters(seed=0)
    return model


def build_sequences(args, vocab):
    if args.dataset != "synthetic":
        return torch.load(args.dataset)
    spec = {"lognormal": LengthSpec("lognormal", lo=16, median=1024.0, sigma=1.2, cap=min(16384, args.max_token_len)),
            "longtail": LengthSpec("longtail", long=(8192, min(32768, args.max_token_len))),
            "uniform": LengthSpec("uniform", lo=64, hi=2048)}[args.length_dist]
    rng = np.random.default_rng(0)  # the same global dataset on every rank; packing decides who gets what
    lens = sample_lengths(spec, args.num_sequences, rng)
    return [torch.from_numpy(rng.integers(0, vocab, size=n)) for n in lens]


def make_dataset(args, cfg, rank, world, odc_enabled):
    seqs = build_sequences(args, cfg.vocab_size)
    kw = {}
    if args.cost_model == "flops":
        h, f = cfg.hidden_size, cfg.intermediate_size
        kw = dict(linear_params=cfg.num_layers * (cfg.qkv_dim * h + h * cfg.num_heads * cfg.head_dim + 3 * h * f),
                  attn_width=cfg.num_layers * cfg.num_heads * cfg.head_dim)
    cost = get_cost_fn(args.cost_model, **kw)
    return BatchedDataset(seqs, args.minibatch_size, rank, world, args.packing_method, args.max_token_len,
                          args.limit_dataset_token_len, cost, odc_enabled)


def microbatch_loss(args, model, mb):
    """Loss of one packed microbatch through the head ``--loss-head`` names (same value either way)."""
    a = (mb["input_ids"], mb["position_ids"], mb["cu_seqlens"], mb["max_seqlen"])
    if getattr(args, "loss_head", "ce") == "logprobs":
        logp = model(*a, labels=mb["labels"], return_logprobs=True)
        return -(logp * mb["loss_scale"].float()).sum()
    return model(*a, labels=mb["labels"], loss_scale=mb["loss_scale"])


_wandb_run = None


def init_logging(args, rank):
    """``ODC_WANDB=1`` and an importable ``wandb``: rank 0 also logs every minibatch's metrics there (project and
    run name from ``--project_name`` / ``--run_name``), as the reference's trainers do."""
    global _wandb_run
    if rank != 0 or os.environ.get("ODC_WANDB", "0") != "1":
        return
    try:
        import wandb
        _wandb_run = wandb.init(project=args.project_name, name=args.run_name, config=vars(args))
    except Exception as e:  # not installed, no API key, no network: training goes on with stdout metrics
        print(f"ODC_WANDB=1 but wandb is unavailable ({type(e).__name__}): metrics go to stdout only", flush=True)
        _wandb_run = None


def log_metrics(rank, step, metrics):
    """Rank 0 prints one JSON line per minibatch (and mirrors it to wandb when :func:`init_logging` set that up)."""
    if rank == 0:
        print(json.dumps({"step": step, **{k: (round(v, 5) if isinstance(v, float) else v) for k, v in metrics.items()}}),
              flush=True)
        if _wandb_run is not None:
            _wandb_run.log(dict(metrics), step=step)


def log_packing(dataset, rank):
    """``ODC_DEBUG_PACKING=1``: every rank's microbatch composition of the last minibatch, printed by rank 0."""
    if os.environ.get("ODC_DEBUG_PACKING", "0") != "1":
        return
    import torch.distributed as dist
    lines = [None] * dist.get_world_size()
    dist.all_gather_object(lines, dataset.last_debug)
    if rank == 0:
        print("\n".join(lines), flush=True)


def memory_metrics():
    if not torch.cuda.is_available():
        return {}
    from odc_b200.runtime.registry import SymmBufferRegistry
    symm = SymmBufferRegistry.get_instance().memory_allocated() / 2**30 if SymmBufferRegistry.is_initialized() else 0.0
    return {"torch_mem_gib": torch.cuda.memory_allocated() / 2**30, "peak_mem_gib": torch.cuda.max_memory_allocated() / 2**30,
            "symm_mem_gib": symm}


def open_checkpoint(args):
    """``--checkpoint-dir``: the checkpoint folder handle (``None`` without the flag)."""
    if not args.checkpoint_dir:
        return None
    from odc_b200.utils.checkpoint import Checkpointer
    return Checkpointer(args.checkpoint_dir)


def maybe_save(args, ck, model, opt, next_step, last):
    """Save after every ``--checkpoint-every`` minibatches and after the last one (collective)."""
    if ck is None or args.forward_only:
        return
    if last or (args.checkpoint_every > 0 and next_step % args.checkpoint_every == 0):
        ck.save(model, opt, meta={"next_step": next_step})


def run_guarded(rank, body):
    """Run the training loop; a peer that left or a wait that ran out ends this rank with exit code 75 (temporary
    failure) and one JSON line, so that a launcher can restart the job, which resumes from ``--checkpoint-dir``."""
    from odc_b200.runtime.status import OdcTimeoutError, PeerFailure
    try:
        return body()
    except (PeerFailure, OdcTimeoutError) as e:
        print(json.dumps({"event": "failure", "rank": rank, "kind": type(e).__name__, "message": str(e)[:300]}), flush=True)
        os._exit(75)   # no collective shutdown: the peers are not all there


def inject_leave(rank, step):
    """Failure drill, made on the host: ``ODC_INJECT_LEAVE="<rank>:<step>"`` lets that rank leave the job right before
    that minibatch, between steps, with nothing of its own in flight.  The others report it (``run_guarded``)."""
    spec = os.environ.get("ODC_INJECT_LEAVE")
    if not spec or os.environ.get("ODC_LAUNCH_ATTEMPT", "0") != "0":
        return   # only the first attempt of a job leaves; one that launch.sh restarted runs through
    r, s = (int(x) for x in spec.split(":"))
    if r == rank and s == step:
        from odc_b200.runtime import control
        hb = control.heartbeat()
        if hb is not None:
            hb.mark_leaving()
        print(json.dumps({"event": "leaving", "rank": rank, "step": step}), flush=True)
        os._exit(0)


def export_model(args, model, cfg):
    """``--save-hf-checkpoint``: the trained weights as a Hugging Face checkpoint folder (collective)."""
    if args.save_hf_checkpoint:
        from odc_b200.utils.checkpoint import Checkpointer
        Checkpointer(args.save_hf_checkpoint).export_hf(model, cfg, args.save_hf_checkpoint)


def mark_done(args):
    out_dir = os.environ.get("ODC_OUT_DIR", "bench_out")
    os.makedirs(out_dir, exist_ok=True)
    with open(os.path.join(out_dir, f"{args.run_name}.done"), "w") as f:
        f.write("done\n")
