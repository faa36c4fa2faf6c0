"""Toy Transformer under FSDP2 with or without on-demand communication.

Counterpart of the reference's examples/FSDP2/example.py: environment switches ``ODC``, ``HPZ``,
``HSDP``; flags ``--explicit-prefetching``, ``--mixed-precision``, ``--dcp-api``;
``ODC_DEBUG_NUMERIC_CORRECTNESS=1`` prints a hash of every gradient gathered on rank 0.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/FSDP2/example.py
    ODC=0 ... (stock FSDP2)   HPZ=1 ...   HSDP=1 ...   (CPU: add --cpu and use the gloo backend)
"""
import argparse
import os
import sys

import torch
import torch.distributed as dist
from torch.distributed.device_mesh import init_device_mesh
from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import odc_b200 as odc  # noqa: E402
from odc_b200.fsdp import fsdp2  # noqa: E402
from odc_b200.models import ToyConfig, ToyTransformer  # noqa: E402
from odc_b200.utils.checkpoint import Checkpointer  # noqa: E402

ODC = os.environ.get("ODC", "1") == "1"
HPZ = os.environ.get("HPZ", "0") == "1"
HSDP = os.environ.get("HSDP", "0") == "1"


def grad_hash(t: torch.Tensor) -> int:
    """Order-stable 31-bit LCG hash of a tensor's bit pattern (cross-rank gradient comparison)."""
    x = t.detach().float().contiguous().view(torch.int32).cpu().to(torch.int64).flatten()
    h = 0
    for chunk in x.split(1 << 16):
        h = (h * 1103515245 + int(chunk.sum()) + 12345) % (1 << 31)
    return h


def set_modules_to_prefetch(model, num_fwd=2, num_bwd=2):
    layers = list(model.layers)
    for i, layer in enumerate(layers):
        layer.set_modules_to_forward_prefetch(layers[i + 1:i + 1 + num_fwd])
        layer.set_modules_to_backward_prefetch(layers[max(0, i - num_bwd):i][::-1])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--explicit-prefetching", action="store_true")
    ap.add_argument("--mixed-precision", action="store_true")
    ap.add_argument("--dcp-api", action="store_true")
    ap.add_argument("--cpu", action="store_true")
    ap.add_argument("--checkpoint-dir", default="")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if args.cpu:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    else:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dev = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group("nccl", device_id=dev)
    if ODC:
        odc.init_nvshmem(dev)
        fsdp2.patch_fsdp2(enable_hpz=HPZ)
    torch.manual_seed(0)
    cfg = ToyConfig(vocab_size=1024, max_seq_len=64, dim=256, n_layers=4, n_heads=8)
    model = ToyTransformer(cfg).to(dev)
    if HSDP:
        mesh = init_device_mesh(dev.type, (2, world // 2), mesh_dim_names=("dp_replicate", "dp_shard"))
    else:
        mesh = init_device_mesh(dev.type, (world,))
    kw = {"mesh": mesh}
    if args.mixed_precision:
        kw["mp_policy"] = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    raf = max(1, (world // 2 if not HSDP else world // 4)) if HPZ else True
    for layer in model.layers:
        fully_shard(layer, reshard_after_forward=raf, **kw)
    fully_shard(model, reshard_after_forward=raf, **kw)
    if args.explicit_prefetching:
        set_modules_to_prefetch(model)
    ck = Checkpointer(args.checkpoint_dir, dcp_api=args.dcp_api) if args.checkpoint_dir else None
    if ck is not None and not ck.is_empty():
        ck.load_model(model)
    if ODC:
        for m in list(model.layers) + [model]:
            fsdp2.patch_lazy_init(m)
    opt = torch.optim.Adam(model.parameters(), lr=1e-2)
    if ck is not None and not ck.is_empty():
        ck.load_optim(model, opt)
    for step in range(10):
        if ODC:
            fsdp2.pre_minibatch_start(model)
        n_micro = 2 + (rank % 2 if ODC else 0)  # on-demand mode tolerates different counts per rank
        for _ in range(n_micro):
            tokens = torch.randint(0, cfg.vocab_size, (8, cfg.max_seq_len), device=dev)
            logits = model(tokens)
            loss = torch.nn.functional.cross_entropy(logits[:, :-1].flatten(0, 1).float(), tokens[:, 1:].flatten())
            loss.backward()
        if ODC:
            fsdp2.pre_optimizer_step(model)
        torch.nn.utils.clip_grad_norm_(model.parameters(), max_norm=1.0)
        if os.environ.get("ODC_DEBUG_NUMERIC_CORRECTNESS", "0") == "1":
            hashes = [grad_hash(p.grad.to_local()) for p in model.parameters() if p.grad is not None]
            gathered = [None] * world
            dist.all_gather_object(gathered, hashes)
            if rank == 0:
                print(f"step {step} grad hashes {[h[:3] for h in gathered]}")
        opt.step()
        opt.zero_grad()
        if rank == 0:
            print(f"step {step} loss {float(loss):.4f}", flush=True)
    if ck is not None:
        ck.save(model, opt)
    if ODC:
        if rank == 0:
            print("symmetric memory (GiB):", fsdp2.get_symm_buffer_memory_breakdown())
        fsdp2.stop()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
