"""Gated delta rule forward on the tcgen05 kernels against the O(T) recurrent definition in fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(B, T, H, seed, strong=False):
    g = torch.Generator(device="cuda").manual_seed(seed)
    q, k, v = (torch.randn(B, T, H, 128, device="cuda", generator=g).bfloat16() for _ in range(3))
    decay = -torch.rand(B, T, H, device="cuda", generator=g) * (2.0 if strong else 0.1)
    beta = torch.rand(B, T, H, device="cuda", generator=g)
    return q, k, v, decay, beta


@pytest.mark.parametrize("B,T,H,strong", [(1, 64, 1, False), (2, 256, 3, False), (1, 200, 2, True)])
def test_gdn_forward_matches_recurrence(B, T, H, strong):
    from archlab_b200.ops import delta_rule as dr
    from archlab_b200.ops import native

    q, k, v, decay, beta = _inputs(B, T, H, 0, strong)
    o, s = dr.gdn_forward_cuda(q, k, v, decay, beta, output_final_state=True)
    torch.cuda.synchronize()
    native.check_status()
    ref = dr.gated_delta_reference(q.float(), k.float(), v.float(), decay, beta)
    _, sref = dr.chunk_gated_delta_rule(q.float(), k.float(), v.float(), decay, beta, output_final_state=True)
    assert (o.float() - ref).norm() / ref.norm() < 2e-2
    assert (s - sref).norm() / sref.norm() < 2e-2


def test_gdn_initial_state_continues_a_sequence():
    from archlab_b200.ops import delta_rule as dr

    q, k, v, decay, beta = _inputs(1, 256, 2, 1)
    full = dr.gdn_forward_cuda(q, k, v, decay, beta)
    h = 128
    o1, s1 = dr.gdn_forward_cuda(q[:, :h], k[:, :h], v[:, :h], decay[:, :h], beta[:, :h], output_final_state=True)
    o2 = dr.gdn_forward_cuda(q[:, h:], k[:, h:], v[:, h:], decay[:, h:], beta[:, h:], initial_state=s1)
    got = torch.cat([o1, o2], 1).float()
    assert (got - full.float()).norm() / full.float().norm() < 1e-2


def test_gdn_autograd_dispatch():
    from archlab_b200.ops import delta_rule as dr

    q, k, v, decay, beta = _inputs(1, 128, 2, 2)
    leaves = [t.clone().requires_grad_(True) for t in (q, k, v, decay, beta)]
    o = dr.gated_delta_rule(*leaves)
    w = torch.randn_like(o, dtype=torch.float32)
    (o.float() * w).sum().backward()
    ref_leaves = [t.detach().float().requires_grad_(True) for t in (q, k, v, decay, beta)]
    (dr.gated_delta_reference(*ref_leaves) * w).sum().backward()
    for a, b in zip(leaves, ref_leaves):
        assert (a.grad.float() - b.grad).norm() / b.grad.norm().clamp_min(1e-9) < 5e-2
