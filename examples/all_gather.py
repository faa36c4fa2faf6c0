"""`gather` against NCCL `all_gather_into_tensor` (counterpart of the reference's examples/all_gather.py).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/all_gather.py [--size-min=65536 --size-max=1073741824]

Every rank owns a bf16 shard of N(0,1) values in the symmetric heap and pulls all peers' shards.
Payload per rank = shard_bytes * (W-1) crosses NVLink inbound; bandwidth = payload / device time
(max over ranks).  Results are checked bitwise against the NCCL output.

With ``--peers=random`` every consumer instead pulls the shards of 1 to W-1 randomly chosen peers (a different
subset and order per rank, size and trial; no collective can express that): the row reports the mean number
of peers, the slowest rank's time and the aggregate inbound rate over all ranks.
"""
import random
import sys

import torch
import torch.distributed as dist

from _prim_bench import NVLINK_GBS, device_time_ms, emit, setup, sizes_from_argv, sync


def random_subsets(g, reg, rank, world, dev):
    rows = []
    for nbytes in sizes_from_argv():
        n = nbytes // 2
        shard = reg.allocate_symm_buffer(f"r{nbytes}", (n,), torch.bfloat16)
        shard.copy_(torch.randn(n, device=dev).bfloat16())
        sync(); dist.barrier()
        ref = torch.empty(world * n, dtype=torch.bfloat16, device=dev)
        dist.all_gather_into_tensor(ref, shard)
        rng = random.Random(1000 * rank + nbytes % 997)
        others = [r for r in range(world) if r != rank]
        trials = [rng.sample(others, rng.randint(1, len(others))) for _ in range(4)]
        times, pulled = [], []
        for peers in trials:
            out = torch.empty(len(peers) * n, dtype=torch.bfloat16, device=dev)
            iters = 10 if nbytes <= (128 << 20) else 4
            times.append(device_time_ms(lambda: g.gather_ranks(out, shard, peers), iters))
            want = torch.cat([ref.view(world, n)[r] for r in peers])
            assert torch.equal(out, want), f"subset gather mismatch at {nbytes} bytes from {peers}"
            pulled.append(len(peers))
            del out, want
        # device_time_ms already takes the max over ranks of each trial; bytes are summed over ranks
        total = torch.tensor([float(sum(pulled)) * nbytes], dtype=torch.float64, device=dev)
        dist.all_reduce(total)
        t = sum(times)
        row = dict(op="gather_subsets", world=world, shard_bytes=nbytes, mean_peers=sum(pulled) / len(pulled), ms=t / len(times),
                   aggregate_gbs=float(total) / t / 1e6, per_rank_gbs=float(total) / world / t / 1e6)
        rows.append(row)
        if rank == 0:
            print(f"gather subsets W={world} shard {nbytes / 2**20:9.3f} MiB, rank 0 pulled {pulled} peers: "
                  f"{row['ms']:8.3f} ms/call (slowest rank), {row['per_rank_gbs']:7.1f} GB/s inbound per rank on average", flush=True)
        reg.deallocate_symm_buffer(f"r{nbytes}")
        del ref
    return rows


def main():
    rank, world, dev = setup()
    import odc_b200 as odc
    reg = odc.init_nvshmem(dev)
    g = odc.GatherService()
    if "--peers=random" in sys.argv:
        emit(rank, random_subsets(g, reg, rank, world, dev), f"gather_subsets_w{world}.json")
        odc.finalize_distributed()
        dist.destroy_process_group()
        return
    rows = []
    for nbytes in sizes_from_argv():
        n = nbytes // 2
        shard = reg.allocate_symm_buffer(f"s{nbytes}", (n,), torch.bfloat16)
        shard.copy_(torch.randn(n, device=dev).bfloat16())
        sync(); dist.barrier()
        out = torch.empty(world * n, dtype=torch.bfloat16, device=dev)
        ref = torch.empty_like(out)
        iters = 20 if nbytes <= (128 << 20) else 8
        t_odc = device_time_ms(lambda: g.gather_into_tensor(out, shard), iters)
        t_nccl = device_time_ms(lambda: dist.all_gather_into_tensor(ref, shard), iters)
        assert torch.equal(out, ref), f"gather mismatch at {nbytes} bytes"
        payload = nbytes * (world - 1)
        row = dict(op="gather", world=world, shard_bytes=nbytes, ms=t_odc, gbs=payload / t_odc / 1e6,
                   nccl_ms=t_nccl, nccl_gbs=payload / t_nccl / 1e6, frac_of_nvlink=payload / t_odc / 1e6 / NVLINK_GBS)
        rows.append(row)
        if rank == 0:
            print(f"gather  W={world} shard {nbytes / 2**20:9.3f} MiB: {t_odc:8.3f} ms {row['gbs']:7.1f} GB/s "
                  f"({row['frac_of_nvlink']:.2f} of {NVLINK_GBS:.0f} GB/s measured link) | NCCL {t_nccl:8.3f} ms {row['nccl_gbs']:7.1f} GB/s", flush=True)
        reg.deallocate_symm_buffer(f"s{nbytes}")
        del out, ref
    emit(rank, rows, f"gather_w{world}.json")
    odc.finalize_distributed()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
