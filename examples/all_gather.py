"""`gather` against NCCL `all_gather_into_tensor` (counterpart of the reference's examples/all_gather.py).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/all_gather.py [--size-min=65536 --size-max=1073741824]

Every rank owns a bf16 shard of N(0,1) values in the symmetric heap and pulls all peers' shards.
Payload per rank = shard_bytes * (W-1) crosses NVLink inbound; bandwidth = payload / device time
(max over ranks).  Results are checked bitwise against the NCCL output.
"""
import torch
import torch.distributed as dist

from _prim_bench import NVLINK_GBS, device_time_ms, emit, setup, sizes_from_argv, sync


def main():
    rank, world, dev = setup()
    import odc_b200 as odc
    reg = odc.init_nvshmem(dev)
    g = odc.GatherService()
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
