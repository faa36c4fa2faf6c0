"""Fused compute+collective kernels against "library GEMM + NCCL collective" (launch with torch.distributed.run).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 examples/bench_fused.py

(1) gather -> GEMM: Y = X W^T, W row-sharded.  Ours: one kernel.  Baseline: NCCL all_gather_into_tensor
    then torch.matmul (cuBLAS).  Roofline time = max(FLOPs / measured bf16 peak, inbound bytes / link).
(1b) gather -> input gradient: dX = dY W with the same sharded W (the gathered rows are the reduction dimension).
(2) wgrad -> scatter-accumulate: dW = dY^T X reduced into the owners' fp32 shards.  Ours: one kernel
    (+ arrival wait).  Baseline: torch.matmul, NCCL reduce_scatter_tensor (fp32), add_.
Device-timed with CUDA events, max over ranks, median of the timed iterations.
"""
import json
import os

import torch
import torch.distributed as dist

from _prim_bench import NVLINK_GBS, device_time_ms, emit, setup


def main():
    rank, world, dev = setup()
    import odc_b200 as odc
    from odc_b200.ops import fused
    peaks_path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    peak_tf, kind = (json.load(open(peaks_path))["bf16_tflops"], "measured") if os.path.exists(peaks_path) else (1590.0, "fallback")
    reg = odc.init_nvshmem(dev)
    red = odc.ReductionService(accumulation_dtype=torch.float32)
    rows = []
    shapes = [(2048, 3072, 2048), (16384, 3072, 2048), (16384, 16384, 2048), (4096, 28672, 4096), (1024, 16384, 2048)]
    for (M, N, K) in shapes:
        rows_per = (N + world - 1) // world
        shard = reg.allocate_symm_buffer(f"w{M}x{N}x{K}", (rows_per, K), torch.bfloat16)
        shard.copy_(0.02 * torch.randn(rows_per, K, device=dev))
        x = torch.randn(M, K, device=dev).bfloat16()
        torch.cuda.synchronize(); dist.barrier()
        w_full = torch.empty(world * rows_per, K, dtype=torch.bfloat16, device=dev)

        def base_fwd():
            dist.all_gather_into_tensor(w_full, shard)
            return torch.matmul(x, w_full[:N].t())

        t_f = device_time_ms(lambda: fused.gather_linear(x, shard, N), 10)
        t_b = device_time_ms(base_fwd, 10)
        y, wf = fused.gather_linear(x, shard, N)
        torch.testing.assert_close(y.float(), base_fwd().float(), rtol=2e-2, atol=2e-1)
        flops = 2.0 * M * N * K
        inbound = rows_per * K * 2 * (world - 1)
        roof_ms = max(flops / (peak_tf * 1e12), inbound / (NVLINK_GBS * 1e9)) * 1e3
        r1 = dict(op="gather_gemm", world=world, M=M, N=N, K=K, ms=t_f, baseline_ms=t_b, roofline_ms=roof_ms,
                  frac_of_roofline=roof_ms / t_f)
        dy = torch.randn(M, N, device=dev).bfloat16()
        # input gradient: dX = dY W with W pulled again (same bytes and FLOPs as the forward product)

        def base_dgrad():
            dist.all_gather_into_tensor(w_full, shard)
            return torch.matmul(dy, w_full[:N])

        t_d = device_time_ms(lambda: fused.gather_dgrad(dy, shard, N), 10)
        t_db = device_time_ms(base_dgrad, 10)
        torch.testing.assert_close(fused.gather_dgrad(dy, shard, N)[0].float(), base_dgrad().float(), rtol=2e-2, atol=2e-1)
        r3 = dict(op="gather_dgrad", world=world, M=M, N=N, K=K, ms=t_d, baseline_ms=t_db, roofline_ms=roof_ms,
                  frac_of_roofline=roof_ms / t_d)
        # weight gradient
        key = f"g{M}x{N}x{K}"
        red.register(key, rows_per * K, torch.float32)
        ref_acc = torch.zeros(rows_per * K, device=dev)
        rs_out = torch.empty(rows_per * K, device=dev)
        pad = world * rows_per - N

        REP = 4  # several microbatches per synchronisation, as in training

        def ours_bwd():
            for _ in range(REP):
                fused.wgrad_scatter(dy, x, red, key, 0, rows_per)
            red.sync()

        def base_bwd():
            for _ in range(REP):
                dw = torch.matmul(dy.t(), x).float()
                if pad:
                    dw = torch.cat([dw, dw.new_zeros(pad, K)])
                dist.reduce_scatter_tensor(rs_out, dw.view(-1))
                ref_acc.add_(rs_out)

        t_f2 = device_time_ms(ours_bwd, 6) / REP
        t_b2 = device_time_ms(base_bwd, 6) / REP
        outbound = rows_per * K * 4 * (world - 1)
        roof2 = max(flops / (peak_tf * 1e12), outbound / (NVLINK_GBS * 1e9)) * 1e3
        r2 = dict(op="wgrad_scatter", world=world, M=M, N=N, K=K, ms=t_f2, baseline_ms=t_b2, roofline_ms=roof2,
                  frac_of_roofline=roof2 / t_f2)
        rows += [r1, r3, r2]
        if rank == 0:
            print(f"W={world} M={M} N={N} K={K}: gather+GEMM {t_f:.3f} ms (NCCL AG + cuBLAS {t_b:.3f} ms; roofline {roof_ms:.3f} ms -> {roof_ms / t_f:.2f} of {kind}) | "
                  f"gather+dgrad {t_d:.3f} ms (NCCL AG + cuBLAS {t_db:.3f} ms -> {roof_ms / t_d:.2f}) | "
                  f"wgrad+scatter {t_f2:.3f} ms (cuBLAS + NCCL RS + add {t_b2:.3f} ms; roofline {roof2:.3f} ms -> {roof2 / t_f2:.2f})", flush=True)
        del x, dy, w_full, ref_acc, rs_out
    emit(rank, rows, f"fused_w{world}.json")
    red.stop()
    odc.finalize_distributed()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
