"""Varlen causal attention kernels against the fp32 PyTorch statement of the op."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(lens, hq, hkv, d, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    T = sum(lens)
    width = (hq + 2 * hkv) * d
    qkv = torch.randn(T, width, device="cuda", generator=g).bfloat16()
    q = qkv[:, : hq * d].view(T, hq, d)
    k = qkv[:, hq * d:(hq + hkv) * d].view(T, hkv, d)
    v = qkv[:, (hq + hkv) * d:].view(T, hkv, d)
    cu = torch.tensor([0] + lens, device="cuda").cumsum(0).int()
    return q, k, v, cu


@pytest.mark.parametrize("lens,hq,hkv,d", [([128], 1, 1, 64), ([256], 2, 1, 64), ([100, 29, 300], 4, 2, 64),
                                           ([128], 1, 1, 128), ([513, 7, 1000, 128], 8, 2, 128),
                                           ([2048, 77], 4, 4, 64)])
def test_attention_forward(lens, hq, hkv, d):
    from odc_b200 import _ext
    from odc_b200.ops import reference as ref
    ext = _ext.load()
    q, k, v, cu = _case(lens, hq, hkv, d)
    o, lse = ext.attn_fwd(q, k, v, cu, max(lens), True, d ** -0.5)
    torch.cuda.synchronize()
    assert ext.kernel_status()[0].item() == 0, ext.kernel_status().tolist()
    want = ref.varlen_attention(q.float(), k.float(), v.float(), cu.cpu(), True, d ** -0.5)
    torch.testing.assert_close(o.float(), want, rtol=2e-2, atol=2e-2)
    # log-sum-exp of the first sequence, first head
    L = lens[0]
    s = (q[:L, 0].float() @ k[:L, 0].float().t()) * d ** -0.5
    s = s.masked_fill(~torch.ones(L, L, dtype=torch.bool, device="cuda").tril(), float("-inf"))
    torch.testing.assert_close(lse[0, :L], torch.logsumexp(s, -1), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("lens,hq,hkv,d", [([128], 1, 1, 64), ([256], 2, 1, 64), ([100, 29, 300], 4, 2, 64),
                                           ([128], 1, 1, 128), ([513, 7, 1000, 128], 8, 2, 128)])
def test_attention_backward(lens, hq, hkv, d):
    from odc_b200 import ops
    from odc_b200.ops import reference as ref
    q, k, v, cu = _case(lens, hq, hkv, d, seed=3)
    q, k, v = (t.detach().clone().requires_grad_() for t in (q, k, v))
    o = ops.varlen_attention(q, k, v, cu, max(lens))
    do = torch.randn_like(o)
    o.backward(do)
    from odc_b200 import _ext
    assert _ext.load().kernel_status()[0].item() == 0
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    want = ref.varlen_attention(qr, kr, vr, cu.cpu(), True, d ** -0.5)
    want.backward(do.float())
    for name, got, exp in (("dq", q.grad, qr.grad), ("dk", k.grad, kr.grad), ("dv", v.grad, vr.grad)):
        err = (got.float() - exp).abs().max().item()
        ref_mag = exp.abs().max().item()
        assert err <= 3e-2 * max(ref_mag, 1.0), (name, err, ref_mag)


def test_attention_on_fused_qkv_matches_reference():
    from odc_b200 import ops
    from odc_b200.ops import reference as ref
    lens, hq, hkv, d = [300, 129, 700], 8, 2, 64
    T = sum(lens)
    cu = torch.tensor([0] + lens, device="cuda").cumsum(0).int()
    qkv = torch.randn(T, (hq + 2 * hkv) * d, device="cuda").bfloat16().requires_grad_()
    o = ops.varlen_attention_qkv(qkv, hq, hkv, d, cu, max(lens))
    do = torch.randn_like(o)
    o.backward(do)
    x = qkv.detach().float().requires_grad_()
    q, k, v = x.split([hq * d, hkv * d, hkv * d], dim=-1)
    want = ref.varlen_attention(q.reshape(T, hq, d), k.reshape(T, hkv, d), v.reshape(T, hkv, d), cu.cpu(), True, d ** -0.5)
    want.backward(do.float())
    torch.testing.assert_close(o.float(), want, rtol=2e-2, atol=2e-2)
    err = (qkv.grad.float() - x.grad).abs().max().item()
    assert err <= 3e-2 * max(x.grad.abs().max().item(), 1.0), err
