"""OdcLinear (fused gather-GEMM / wgrad-scatter layer) on CPU ranks: same result as a dense layer."""
import pytest
import torch

from _mp import run_ranks


def _run(rank, world, keep_weight):
    import odc_b200 as odc
    from odc_b200 import parallel
    odc.init_nvshmem("cpu", 64 << 20)
    lin = parallel.OdcLinear(32, 50, seed=3, keep_weight=keep_weight)
    torch.manual_seed(100 + rank)
    xs = [torch.randn(7 + rank, 32, requires_grad=True) for _ in range(1 + rank)]  # uneven microbatch counts
    parallel.start_minibatch()
    ys = []
    for x in xs:
        y = lin(x)
        y.pow(2).sum().backward()
        ys.append(y.detach())
    from odc_b200.runtime import control
    shard_before = lin.weight.master.clone()
    parallel.finish_minibatch(lr=0.0)  # sync only; lr 0 keeps the weights so the gradient can be checked
    grad = lin.weight.grad().clone()
    out = dict(xs=[x.detach() for x in xs], dxs=[x.grad for x in xs], ys=ys, grad=grad, shard=shard_before,
               rows=lin.weight.rows_per_rank)
    control.host_barrier()
    parallel.reset()
    odc.finalize_distributed()
    return out


@pytest.mark.parametrize("keep_weight", [False, True])
def test_odc_linear_matches_dense(keep_weight):
    world = 2
    res = run_ranks(_run, world, keep_weight)
    W = torch.cat([r["shard"] for r in res])[:50]
    Wb = W.bfloat16().float()  # peers pull the bf16 copy
    dW = torch.zeros(50, 32)
    for r in res:
        for x, y, dx in zip(r["xs"], r["ys"], r["dxs"]):
            want = x @ Wb.t()
            torch.testing.assert_close(y, want, rtol=1e-4, atol=1e-4)
            torch.testing.assert_close(dx, (2 * want) @ Wb, rtol=1e-4, atol=1e-4)
            dW += (2 * want).t() @ x
    dW /= world
    got = torch.cat([r["grad"] for r in res])[:50]
    torch.testing.assert_close(got, dW, rtol=1e-4, atol=1e-4)
