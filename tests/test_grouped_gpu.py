"""Grouped expert GEMM (one launch, per-tile expert table) against per-expert fp32 products, with gradients."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_grouped_linear_forward_backward():
    from archlab_b200.ops import grouped, native

    torch.manual_seed(0)
    E, N, K = 4, 384, 256
    real = [300, 0, 513, 40]
    padded = [int(v) for v in grouped.padded_sizes(torch.tensor(real))]
    assert padded == [512, 0, 768, 256]
    tiles = grouped.tile_groups(padded, "cuda")
    assert tiles.tolist() == [0, 0, 2, 2, 2, 3]
    x = (torch.randn(sum(padded), K, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(E, N, K, device="cuda") * 0.1).bfloat16().requires_grad_(True)
    y = grouped.grouped_linear(x, w, tiles, real, padded)
    mask = torch.zeros(sum(padded), 1, device="cuda")
    s0 = 0
    for n, npad in zip(real, padded):
        mask[s0:s0 + n] = 1
        s0 += npad
    g = torch.randn_like(y, dtype=torch.float32) * mask                 # nothing flows back from padding rows
    (y.float() * g).sum().backward()
    native.check_status()
    xf, wf = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    outs, s0 = [], 0
    for e, npad in enumerate(padded):
        outs.append(xf[s0:s0 + npad] @ wf[e].t())
        s0 += npad
    yr = torch.cat(outs)
    (yr * g).sum().backward()
    rel = lambda a, b: ((a.float() - b) * 1).norm() / b.norm()
    assert rel(y.float() * mask, yr * mask) < 1e-2
    assert rel(x.grad.float() * mask, xf.grad * mask) < 2e-2 and rel(w.grad, wf.grad) < 2e-2
