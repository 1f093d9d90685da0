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
