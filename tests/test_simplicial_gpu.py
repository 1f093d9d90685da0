"""sm_100a 2-simplicial attention kernel against the fp32 PyTorch statement (the ladder of window
shapes follows the reference's preflight, src/archlab/qualification/simplicial_attention.py:196-215)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,N,Hq,Hkv,w1,w2", [(1, 64, 1, 1, 8, 8), (1, 130, 2, 1, 16, 64), (2, 300, 2, 2, 32, 128),
                                               (1, 529, 2, 1, 32, 512), (1, 257, 4, 2, 16, 128)])
def test_simplicial_forward(B, N, Hq, Hkv, w1, w2):
    from archlab_b200.ops import native
    from archlab_b200.ops.simplicial import simplicial_attention_reference
    from archlab_b200.ops.simplicial_cuda import simplicial_fwd

    torch.manual_seed(0)
    D = 128
    mk = lambda H: (torch.randn(B, N, H, D, device="cuda") * 0.7).bfloat16()
    q, k1, k2, v1, v2 = mk(Hq), mk(Hkv), mk(Hkv), mk(Hkv), mk(Hkv)
    scale = D ** -0.5
    out, lse2 = simplicial_fwd(q, k1, k2, v1, v2, w1, w2, scale)
    torch.cuda.synchronize()
    native.check_status()
    ref = simplicial_attention_reference(q.float(), k1.float(), k2.float(), v1.float(), v2.float(), w1, w2,
                                         scale=scale)
    rel = ((out.float() - ref).norm() / ref.norm()).item()
    assert rel < 2.5e-2, rel
    assert not torch.isnan(out.float()).any()


@pytest.mark.parametrize("B,N,Hq,Hkv,w1,w2", [(1, 64, 1, 1, 8, 8), (1, 130, 2, 1, 16, 64), (2, 300, 2, 2, 32, 128),
                                               (1, 529, 2, 1, 32, 512), (1, 257, 4, 2, 8, 100)])
def test_simplicial_backward(B, N, Hq, Hkv, w1, w2):
    from archlab_b200.ops import native
    from archlab_b200.ops.simplicial import simplicial_attention_reference
    from archlab_b200.ops.simplicial_bwd import simplicial_bwd
    from archlab_b200.ops.simplicial_cuda import simplicial_fwd

    torch.manual_seed(1)
    D = 128
    mk = lambda H: (torch.randn(B, N, H, D, device="cuda") * 0.7).bfloat16()
    q, k1, k2, v1, v2 = mk(Hq), mk(Hkv), mk(Hkv), mk(Hkv), mk(Hkv)
    dout = (torch.randn(B, N, Hq, D, device="cuda") * 0.3).bfloat16()
    scale = D ** -0.5
    out, lse2 = simplicial_fwd(q, k1, k2, v1, v2, w1, w2, scale)
    got = simplicial_bwd(q, k1, k2, v1, v2, out, dout, lse2, w1, w2, scale)
    torch.cuda.synchronize()
    native.check_status()
    ins = [t.float().requires_grad_(True) for t in (q, k1, k2, v1, v2)]
    ref = simplicial_attention_reference(*ins, w1, w2, scale=scale)
    want = torch.autograd.grad(ref, ins, dout.float())
    for name, g, w in zip(("dq", "dk1", "dk2", "dv1", "dv2"), got, want):
        rel = ((g.float() - w).norm() / w.norm().clamp_min(1e-9)).item()
        assert rel < 3e-2, (name, rel)
        assert torch.isfinite(g.float()).all(), name


@pytest.mark.parametrize("B,N,Hq,Hkv,w1,w2", [(1, 130, 2, 1, 16, 64), (2, 300, 2, 2, 32, 128), (1, 529, 4, 2, 8, 512)])
def test_deterministic_backward_is_bit_reproducible_and_matches_the_oracle(B, N, Hq, Hkv, w1, w2):
    from archlab_b200.ops import native
    from archlab_b200.ops.simplicial import simplicial_attention_reference
    from archlab_b200.ops.simplicial_bwd import simplicial_bwd
    from archlab_b200.ops.simplicial_cuda import simplicial_fwd

    torch.manual_seed(2)
    D = 128
    mk = lambda H: (torch.randn(B, N, H, D, device="cuda") * 0.7).bfloat16()
    q, k1, k2, v1, v2 = mk(Hq), mk(Hkv), mk(Hkv), mk(Hkv), mk(Hkv)
    dout = (torch.randn(B, N, Hq, D, device="cuda") * 0.3).bfloat16()
    scale = D ** -0.5
    out, lse2 = simplicial_fwd(q, k1, k2, v1, v2, w1, w2, scale)
    first = simplicial_bwd(q, k1, k2, v1, v2, out, dout, lse2, w1, w2, scale, deterministic=True)
    again = simplicial_bwd(q, k1, k2, v1, v2, out, dout, lse2, w1, w2, scale, deterministic=True)
    torch.cuda.synchronize()
    native.check_status()
    for name, a, b in zip(("dq", "dk1", "dk2", "dv1", "dv2"), first, again):
        assert torch.equal(a, b), name
    ins = [t.float().requires_grad_(True) for t in (q, k1, k2, v1, v2)]
    want = torch.autograd.grad(simplicial_attention_reference(*ins, w1, w2, scale=scale), ins, dout.float())
    for name, g, w in zip(("dq", "dk1", "dk2", "dv1", "dv2"), first, want):
        assert ((g.float() - w).norm() / w.norm().clamp_min(1e-9)).item() < 3e-2, name
    # the global switch selects the same path
    torch.use_deterministic_algorithms(True, warn_only=True)
    try:
        third = simplicial_bwd(q, k1, k2, v1, v2, out, dout, lse2, w1, w2, scale)
    finally:
        torch.use_deterministic_algorithms(False)
    assert all(torch.equal(a, b) for a, b in zip(first, third))
