"""Memory-bound trunk kernels against fp32 PyTorch autograd on the same bf16 inputs."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def test_mix_norm_and_backward():
    from archlab_b200.ops import trunk

    torch.manual_seed(0)
    R, C = 777, 1280
    x = torch.randn(R, C, device=DEV).bfloat16()
    x0 = torch.randn(R, C, device=DEV).bfloat16()
    a = torch.tensor([1.1], device=DEV)
    b = torch.tensor([0.15], device=DEV)
    x1, n = trunk.mix_norm_fwd(x, x0, a, b)
    xf, x0f = x.float().requires_grad_(True), x0.float().requires_grad_(True)
    af, bf_ = a.clone().requires_grad_(True), b.clone().requires_grad_(True)
    x1r = (af * xf + bf_ * x0f)
    nr = F.rms_norm(x1r.detach().bfloat16().float() + (x1r - x1r.detach()), (C,))
    assert rel(x1, x1r) < 4e-3 and rel(n, nr) < 4e-3
    dn = torch.randn(R, C, device=DEV).bfloat16()
    dres = torch.randn(R, C, device=DEV).bfloat16()
    (nr * dn.float()).sum().backward(retain_graph=True)
    (x1r * dres.float()).sum().backward()
    dx0 = torch.empty_like(x)
    da = torch.zeros(1, device=DEV)
    db = torch.zeros(1, device=DEV)
    dx = trunk.norm_bwd_mix(x1, dn, dres, a, b, x, x0, dx0, True, da, db)
    assert rel(dx, xf.grad) < 6e-3 and rel(dx0, x0f.grad) < 6e-3
    assert abs(da.item() - af.grad.item()) < 2e-2 * (abs(af.grad.item()) + 1.0)
    assert abs(db.item() - bf_.grad.item()) < 2e-2 * (abs(bf_.grad.item()) + 1.0)
    # plain norm backward with residual
    x2 = x.float().requires_grad_(True)
    (F.rms_norm(x2, (C,)) * dn.float()).sum().backward()
    got = trunk.norm_bwd(x, dn, dres)
    assert rel(got, x2.grad + dres.float()) < 6e-3


def test_embed_forward_backward():
    from archlab_b200.ops import trunk

    torch.manual_seed(1)
    V, C, B, T, G = 512, 256, 3, 64, 24
    wte = torch.randn(V, C, device=DEV).bfloat16()
    gate_w = (torch.rand(G, device=DEV) * 0.5)
    lam = torch.tensor([0.4], device=DEV)
    idx = torch.randint(0, V, (B, T), device=DEV)
    x0, gate_pre = trunk.embed_fwd(idx.view(-1), wte, gate_w, lam, T)
    w = wte.float().requires_grad_(True)
    gw = gate_w.clone().requires_grad_(True)
    lm = lam.clone().requires_grad_(True)
    e = F.rms_norm(w[idx], (C,))
    gate = lm * torch.sigmoid(e[:, 1:, :G] @ gw.view(-1, 1))
    ref = torch.cat([e[:, :1], e[:, 1:] + gate * e[:, :-1]], dim=1)
    assert rel(x0.view(B, T, C), ref) < 6e-3
    g = torch.randn(B * T, C, device=DEV).bfloat16()
    (ref * g.view(B, T, C).float()).sum().backward()
    dw = torch.zeros(V, C, device=DEV)
    dgw = torch.zeros(G, device=DEV)
    dl = torch.zeros(1, device=DEV)
    trunk.embed_bwd(idx.view(-1), wte, gate_w, lam, gate_pre, g, dw, dgw, dl, T)
    assert rel(dw, w.grad) < 1e-2
    assert rel(dgw, gw.grad) < 2e-2
    assert abs(dl.item() - lm.grad.item()) < 2e-2 * (abs(lm.grad.item()) + 1.0)


@pytest.mark.parametrize("with_ve", [False, True])
def test_qkv_post_forward_backward(with_ve):
    from archlab_b200.models.nanochat import apply_rope, rotary_tables
    from archlab_b200.ops import trunk

    torch.manual_seed(2)
    B, T, Hq, Hkv, D, C, V, GC = 2, 64, 4, 2, 128, 256, 300, 12
    rows = B * T
    qkv = torch.randn(rows, (Hq + 2 * Hkv) * D, device=DEV).bfloat16()
    n = torch.randn(rows, C, device=DEV).bfloat16()
    idx = torch.randint(0, V, (rows,), device=DEV)
    cos, sin = rotary_tables(T, D, torch.float32, device=DEV)
    ve = torch.randn(V, Hkv * D, device=DEV).bfloat16() if with_ve else None
    gate_w = (torch.rand(Hkv, GC, device=DEV) * 0.3) if with_ve else None
    src = qkv.clone()
    rstd, gate_pre = trunk.qkv_post_fwd(qkv, cos, sin, 1.2, idx, ve, gate_w, n, T, Hq, Hkv, D)
    # reference
    s = src.float().requires_grad_(True)
    q = s[:, :Hq * D].view(B, T, Hq, D)
    k = s[:, Hq * D:(Hq + Hkv) * D].view(B, T, Hkv, D)
    v = s[:, (Hq + Hkv) * D:].view(B, T, Hkv, D)
    qr = F.rms_norm(apply_rope(q, cos, sin), (D,)) * 1.2
    kr = F.rms_norm(apply_rope(k, cos, sin), (D,)) * 1.2
    if with_ve:
        vef = ve.float().requires_grad_(True)
        gwf = gate_w.clone().requires_grad_(True)
        nf = n.float().requires_grad_(True)
        gate = 3 * torch.sigmoid(nf[:, :GC] @ gwf.t())
        v = v + gate.view(B, T, Hkv, 1) * vef[idx].view(B, T, Hkv, D)
    ref = torch.cat([qr.reshape(rows, -1), kr.reshape(rows, -1), v.reshape(rows, -1)], dim=1)
    assert rel(qkv, ref) < 8e-3
    dout = torch.randn_like(qkv)
    (ref * dout.float()).sum().backward()
    dqkv = dout.clone()
    dve = torch.zeros(V, Hkv * D, device=DEV) if with_ve else None
    dgp = trunk.qkv_post_bwd(dqkv, qkv, cos, sin, 1.2, idx, ve, rstd, gate_pre, dve, T, Hq, Hkv, D)
    assert rel(dqkv, s.grad) < 1.2e-2
    if with_ve:
        assert rel(dve, vef.grad) < 1e-2
        dn = torch.zeros(rows, C, device=DEV).bfloat16()
        dgw = torch.zeros(Hkv, GC, device=DEV)
        trunk.gate_bwd(dn, n, dgp, gate_w, dgw)
        assert rel(dgw, gwf.grad) < 2e-2
        assert rel(dn[:, :GC], nf.grad[:, :GC]) < 2e-2


def test_softcap_cross_entropy():
    from archlab_b200.ops import trunk

    torch.manual_seed(3)
    N, V = 300, 4096
    logits = (torch.randn(N, V, device=DEV) * 6).bfloat16()
    tgt = torch.randint(0, V, (N,), device=DEV)
    tgt[::17] = -1
    lf = logits.float().requires_grad_(True)
    z = 15 * torch.tanh(lf / 15)
    loss = F.cross_entropy(z, tgt, ignore_index=-1, reduction="none")
    (loss.sum() * 0.01).backward()
    work = logits.clone()
    rows = trunk.softcap_ce_(work, tgt, 0.01)
    assert rel(rows, loss) < 2e-3
    assert rel(work, lf.grad) < 1e-2
