"""`scatter_accumulate` against NCCL `reduce_scatter_tensor` + `add_` (counterpart of the reference's examples/reduce_scatter.py).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/reduce_scatter.py [--dtype=bf16|fp32]

Each rank adds a [W, shard] tensor into the owners' fp32 accumulators.  Payload per rank =
shard_bytes * (W-1) outbound.  The timed region of the on-demand path includes the arrival wait
(`sync`) so that both sides are timed to "sum complete on the owner".  Inputs are small integers,
so sums are exact and the result is compared bitwise with the NCCL path.
"""
import sys

import torch
import torch.distributed as dist

from _prim_bench import NVLINK_GBS, device_time_ms, emit, reduce_scatter_sum, setup, sizes_from_argv, sync


def main():
    rank, world, dev = setup()
    dtype = torch.float32 if "--dtype=fp32" in sys.argv else torch.bfloat16
    esize = 4 if dtype == torch.float32 else 2
    import odc_b200 as odc
    odc.init_nvshmem(dev)
    red = odc.ReductionService(accumulation_dtype=torch.float32)
    rows = []
    for nbytes in sizes_from_argv(default_hi=512 << 20):
        n = nbytes // esize
        x = torch.randint(-4, 5, (world * n,), device=dev).to(dtype)
        key = f"k{nbytes}"
        red.register(key, n, dtype)
        acc = red.get_accumulation(key)
        ref_acc = torch.zeros(n, device=dev)
        rs_out = torch.empty(n, dtype=dtype, device=dev)
        iters = 10 if nbytes <= (128 << 20) else 5

        def odc_fn():
            red.scatter_accumulate(key, x)
            red.sync()

        def nccl_fn():
            reduce_scatter_sum(rs_out, x)
            ref_acc.add_(rs_out)

        acc.zero_(); ref_acc.zero_(); sync(); dist.barrier()
        t_odc = device_time_ms(odc_fn, iters)
        t_nccl = device_time_ms(nccl_fn, iters)
        sync(); dist.barrier()
        assert torch.equal(acc, ref_acc), f"scatter_accumulate mismatch at {nbytes}: {(acc - ref_acc).abs().max()}"
        payload = nbytes * (world - 1)
        row = dict(op="scatter_accumulate", world=world, dtype=str(dtype), shard_bytes=nbytes, ms=t_odc,
                   gbs=payload / t_odc / 1e6, nccl_ms=t_nccl, nccl_gbs=payload / t_nccl / 1e6,
                   frac_of_nvlink=payload / t_odc / 1e6 / NVLINK_GBS)
        rows.append(row)
        if rank == 0:
            print(f"scatter W={world} {dtype} shard {nbytes / 2**20:9.3f} MiB: {t_odc:8.3f} ms {row['gbs']:7.1f} GB/s "
                  f"({row['frac_of_nvlink']:.2f} of {NVLINK_GBS:.0f} GB/s measured link) | NCCL rs+add {t_nccl:8.3f} ms {row['nccl_gbs']:7.1f} GB/s", flush=True)
        del x, ref_acc, rs_out
    emit(rank, rows, f"scatter_w{world}_{'fp32' if dtype == torch.float32 else 'bf16'}.json")
    red.stop()
    odc.finalize_distributed()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
