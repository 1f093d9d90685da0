"""Fused optimizer kernels against the PyTorch statement of the same update rules."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_fused_adamw_matches_reference():
    from archlab_b200.optim.fused import fused_adamw_
    from archlab_b200.optim.muon import adamw_update

    torch.manual_seed(0)
    n = 4096 * 33
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda") * 0.1
    m = torch.randn(n, device="cuda") * 0.01
    v = torch.rand(n, device="cuda") * 0.01
    shadow = torch.empty(n, dtype=torch.bfloat16, device="cuda")
    for cautious in (False, True):
        pr, mr, vr = p.clone(), m.clone(), v.clone()
        adamw_update(pr, g, mr, vr, step=3, lr=0.01, beta1=0.8, beta2=0.95, eps=1e-10, wd=0.1, cautious=cautious)
        pf, mf, vf = p.clone(), m.clone(), v.clone()
        fused_adamw_(pf, g, mf, vf, shadow, step=3, lr=0.01, beta1=0.8, beta2=0.95, eps=1e-10, wd=0.1,
                     cautious=cautious)
        torch.cuda.synchronize()
        assert torch.allclose(pf, pr, rtol=1e-5, atol=1e-6)
        assert torch.allclose(mf, mr, rtol=1e-5, atol=1e-7) and torch.allclose(vf, vr, rtol=1e-5, atol=1e-8)
        assert torch.equal(shadow, pf.bfloat16())


@pytest.mark.parametrize("shape", [(256, 256), (512, 128), (128, 512)])
def test_fused_muon_matches_reference(shape):
    from archlab_b200.optim.fused import fused_muon_
    from archlab_b200.optim.muon import muon_update

    torch.manual_seed(1)
    K = 3
    m, n = shape
    master = torch.randn(K, m, n, device="cuda") * 0.05
    grad = torch.randn(K, m, n, device="cuda")
    mom = torch.randn(K, m, n, device="cuda") * 0.1
    sshape = (K, m, 1) if m >= n else (K, 1, n)
    sm = torch.rand(sshape, device="cuda") * 0.5 + 0.5
    kw = dict(momentum=0.95, lr=0.02, wd=0.1, beta2=0.9, ns_steps=5)
    pr, gr, mr, smr = master.clone(), grad.clone(), mom.clone(), sm.clone()
    muon_update(gr, pr, mr, smr, red_dim=-1 if m >= n else -2, bf16=True, **kw)
    pf, gf = master.clone(), grad.clone()
    shadow = torch.empty(K, m, n, dtype=torch.bfloat16, device="cuda")
    state = {"momentum_buffer": mom.clone(), "second_momentum_buffer": sm.clone(),
             "norm2": torch.zeros(K, device="cuda")}
    fused_muon_(pf, gf, shadow, state, **kw)
    torch.cuda.synchronize()
    assert torch.allclose(state["momentum_buffer"], mr, rtol=1e-5, atol=1e-6)
    du, dr = pf - master, pr - master
    rel = ((du - dr).norm() / dr.norm()).item()
    assert rel < 3e-2, rel        # both run the Newton-Schulz iteration in bf16
    assert torch.allclose(state["second_momentum_buffer"], smr, rtol=2e-2, atol=1e-4)
    assert torch.equal(shadow, pf.bfloat16())
