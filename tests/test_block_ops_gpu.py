"""Fused RMSNorm / RoPE / SwiGLU / cross-entropy autograd ops against fp32 PyTorch statements."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.mark.parametrize("shape,groups,zero_centered,gain", [((512, 16, 128), 1, False, True), ((300, 2560), 1, False, True),
                                                             ((257, 1024), 4, True, True), ((64, 8192), 1, False, False),
                                                             ((1000, 640), 1, True, True)])
def test_rmsnorm_forward_backward(shape, groups, zero_centered, gain):
    from archlab_b200.ops import block_ops, native

    torch.manual_seed(0)
    x = torch.randn(*shape, device="cuda").bfloat16().requires_grad_(True)
    w = ((torch.randn(shape[-1], device="cuda") * 0.2 + (0 if zero_centered else 1)).requires_grad_(True)) if gain else None
    dy = torch.randn(*shape, device="cuda").bfloat16()
    y = block_ops.rms_norm(x, w, eps=1e-6, zero_centered=zero_centered, groups=groups)
    y.backward(dy)
    xf = x.detach().float().requires_grad_(True)
    wf = w.detach().clone().requires_grad_(True) if gain else None
    xs = xf.unflatten(-1, (groups, shape[-1] // groups))
    yr = xs * torch.rsqrt(xs.square().mean(-1, keepdim=True) + 1e-6)
    yr = yr.flatten(-2)
    if gain:
        yr = yr * ((1 + wf) if zero_centered else wf)
    yr.backward(dy.float())
    native.check_status()
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xf.grad) < 1e-2
    if gain:
        assert _rel(w.grad, wf.grad) < 1e-2


@pytest.mark.parametrize("style,rot", [("half", 128), ("interleaved", 64)])
def test_rope_forward_backward(style, rot):
    from archlab_b200.models.blocks import apply_rope, rope_tables
    from archlab_b200.ops import block_ops

    torch.manual_seed(1)
    x = torch.randn(2, 256, 4, 128, device="cuda").bfloat16().requires_grad_(True)
    cos, sin = rope_tables(256, rot, 10000.0, "cuda")
    dy = torch.randn_like(x)
    y = block_ops.rope(x, cos, sin, rot_dim=rot, interleaved=style == "interleaved")
    y.backward(dy)
    xf = x.detach().float().cpu().requires_grad_(True)
    yr = apply_rope(xf, cos.cpu(), sin.cpu(), style=style, rot_dim=rot)
    yr.backward(dy.float().cpu())
    assert _rel(y.cpu(), yr) < 1e-2 and _rel(x.grad.cpu(), xf.grad) < 1e-2


@pytest.mark.parametrize("limit", [None, 1.5])
def test_swiglu_forward_backward(limit):
    from archlab_b200.ops import block_ops

    torch.manual_seed(2)
    h = (torch.randn(300, 2 * 1408, device="cuda") * 2).bfloat16().requires_grad_(True)
    dy = torch.randn(300, 1408, device="cuda").bfloat16()
    y = block_ops.swiglu(h, limit)
    y.backward(dy)
    hf = h.detach().float().requires_grad_(True)
    g, u = hf.chunk(2, -1)
    if limit is not None:
        g, u = g.clamp(max=limit), u.clamp(-limit, limit)
    yr = F.silu(g) * u
    yr.backward(dy.float())
    assert _rel(y, yr) < 1e-2 and _rel(h.grad, hf.grad) < 1e-2


def test_cross_entropy_sum_inplace_gradient():
    from archlab_b200.ops import block_ops

    torch.manual_seed(3)
    rows, V = 200, 151936
    base = (torch.randn(rows, V, device="cuda") * 3).bfloat16()
    tgt = torch.randint(0, V, (rows,), device="cuda")
    tgt[::7] = -1
    logits = base.clone().requires_grad_(True)
    work = logits * 1.0                                   # a fresh buffer the op may consume
    loss = block_ops.cross_entropy_sum(work, tgt) / 10
    loss.backward()
    lf = base.float().requires_grad_(True)
    lr = F.cross_entropy(lf, tgt, ignore_index=-1, reduction="sum") / 10
    lr.backward()
    assert abs(loss.item() - lr.item()) / lr.item() < 1e-3
    assert _rel(logits.grad, lf.grad) < 1e-2
