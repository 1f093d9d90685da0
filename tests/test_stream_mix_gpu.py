"""Per-token stream mixing kernels (hyper-connection read / write-back) against fp32 einsums."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n,C,tokens", [(4, 2048, 300), (2, 256, 17), (4, 1000, 64)])
def test_hyper_connection_read_write(n, C, tokens):
    from archlab_b200.ops import native, stream_mix as sm

    torch.manual_seed(0)
    streams = torch.randn(3, tokens, n, C, device="cuda").bfloat16().requires_grad_(True)
    y = torch.randn(3, tokens, C, device="cuda").bfloat16().requires_grad_(True)
    pre = torch.rand(3, tokens, n, device="cuda", requires_grad=True)
    post = torch.rand(3, tokens, n, device="cuda", requires_grad=True)
    comb = torch.rand(3, tokens, n, n, device="cuda", requires_grad=True)
    g1, g2 = torch.randn(3, tokens, C, device="cuda"), torch.randn(3, tokens, n, C, device="cuda")
    x = sm.hyper_connection_read(pre, streams)
    out = sm.hyper_connection_write(comb, post, streams, y)
    ((x.float() * g1).sum() + (out.float() * g2).sum()).backward()
    native.check_status()
    leaves = [t.detach().float().requires_grad_(True) for t in (streams, y, pre, post, comb)]
    sf, yf, pf, qf, cf = leaves
    xr = (sf * pf.unsqueeze(-1)).sum(-2)
    outr = cf.transpose(-1, -2) @ sf + qf.unsqueeze(-1) * yf.unsqueeze(-2)
    ((xr * g1).sum() + (outr * g2).sum()).backward()
    rel = lambda a, b: ((a.float() - b).norm() / b.norm().clamp_min(1e-9)).item()
    assert rel(x, xr) < 1e-2 and rel(out, outr) < 1e-2
    for got, want in zip((streams, y, pre, post, comb), leaves):
        assert rel(got.grad, want.grad) < 2e-2


def test_hc_coefficients_kernel_matches_pytorch():
    import torch.nn.functional as F  # noqa: F401

    from archlab_b200.models import blocks
    from archlab_b200.ops import native, stream_mix as sm

    torch.manual_seed(0)
    mixes = torch.randn(3, 50, 24, device="cuda", requires_grad=True)
    scale = torch.tensor([0.5, 0.7, 1.3], device="cuda", requires_grad=True)
    base = (torch.randn(24, device="cuda") * 0.3).requires_grad_(True)
    gp, gq, gc = torch.randn(3, 50, 4, device="cuda"), torch.randn(3, 50, 4, device="cuda"), torch.randn(3, 50, 4, 4, device="cuda")
    pre, post, comb = sm.hc_coefficients(mixes, scale, base, 20, 1e-6)
    ((pre * gp).sum() + (post * gq).sum() + (comb * gc).sum()).backward()
    native.check_status()
    ref = [t.detach().double().cpu().requires_grad_(True) for t in (mixes, scale, base)]
    rp, rq, rc = blocks.hc_split_sinkhorn(ref[0], ref[1], ref[2], 4, 20, 1e-6)
    ((rp * gp.double().cpu()).sum() + (rq * gq.double().cpu()).sum() + (rc * gc.double().cpu()).sum()).backward()
    close = lambda a, b: torch.allclose(a.double().cpu(), b, atol=2e-4, rtol=2e-3)
    assert close(pre, rp) and close(post, rq) and close(comb, rc)
    assert torch.allclose(comb.sum(-2), torch.ones(3, 50, 4, device="cuda"), atol=1e-3)      # columns balanced
    for got, want in zip((mixes, scale, base), ref):
        assert close(got.grad, want.grad), (got.grad.flatten()[:4], want.grad.flatten()[:4])
