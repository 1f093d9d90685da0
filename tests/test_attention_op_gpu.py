"""Autograd attention op over the flash kernels against the fp32 masked-softmax definition."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("Hq,Hkv,window", [(4, 4, -1), (8, 2, -1), (4, 2, 256)])
def test_causal_attention_forward_backward(Hq, Hkv, window):
    from archlab_b200.ops import native, trunk
    from archlab_b200.ops.attention import causal_attention

    torch.manual_seed(0)
    B, T, D = 2, 512, 128
    q = (torch.randn(B, T, Hq, D, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    k = (torch.randn(B, T, Hkv, D, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    v = (torch.randn(B, T, Hkv, D, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w = torch.randn(B, T, Hq, D, device="cuda")
    o = causal_attention(q, k, v, window)
    (o.float() * w).sum().backward()
    got = [o.detach().float(), q.grad.float(), k.grad.float(), v.grad.float()]
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    of = trunk.attention_reference(qf, kf, vf, window)
    (of * w).sum().backward()
    want = [of.detach(), qf.grad, kf.grad, vf.grad]
    native.check_status()
    for g, r in zip(got, want):
        assert (g - r).norm() / r.norm() < 2e-2
