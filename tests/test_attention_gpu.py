"""tcgen05 attention forward / backward against the fp32 masked-softmax definition."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,T,Hq,Hkv,window", [(1, 128, 1, 1, -1), (1, 256, 2, 2, -1), (2, 512, 2, 1, 128),
                                                 (1, 1024, 2, 2, 512), (1, 320, 1, 1, -1), (1, 640, 4, 2, 200)])
def test_attention_fwd_bwd(B, T, Hq, Hkv, window):
    from archlab_b200.ops import native, trunk

    torch.manual_seed(0)
    D = 128
    qkv = torch.randn(B * T, (Hq + 2 * Hkv) * D, device="cuda").bfloat16()
    out, lse2 = trunk.attn_fwd(qkv, B, T, Hq, Hkv, D, window)
    q = qkv[:, :Hq * D].view(B, T, Hq, D).float().requires_grad_(True)
    k = qkv[:, Hq * D:(Hq + Hkv) * D].view(B, T, Hkv, D).float().requires_grad_(True)
    v = qkv[:, (Hq + Hkv) * D:].view(B, T, Hkv, D).float().requires_grad_(True)
    ref = trunk.attention_reference(q, k, v, window)
    torch.cuda.synchronize()
    native.check_status()
    o = out.view(B, T, Hq, D).float()
    assert ((o - ref).norm() / ref.norm()).item() < 5e-3
    do = torch.randn_like(out)
    dqkv = trunk.attn_bwd(qkv, out, do, lse2, B, T, Hq, Hkv, D, window)
    torch.cuda.synchronize()
    native.check_status()
    ref.backward(do.view(B, T, Hq, D).float())
    dq = dqkv[:, :Hq * D].view(B, T, Hq, D).float()
    dk = dqkv[:, Hq * D:(Hq + Hkv) * D].view(B, T, Hkv, D).float()
    dv = dqkv[:, (Hq + Hkv) * D:].view(B, T, Hkv, D).float()
    for got, want in ((dq, q.grad), (dk, k.grad), (dv, v.grad)):
        assert ((got - want).norm() / want.norm()).item() < 8e-3
