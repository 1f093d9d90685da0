"""Frozen V4.1 backbone: input gradients match plain autograd through the same rounded weights, nothing else trains,
and the linears do not keep their input."""
import pytest
import torch

from archlab_b200.models.deepseek_v41 import HyperConnectionMix, QuantLinear, V41Config, V41LM
from archlab_b200.models.v41_frozen import FrozenCoefficientsFn, FrozenLinearFn, freeze_backbone
from archlab_b200.models.blocks import hc_split_sinkhorn


def test_frozen_linear_is_a_straight_through_surrogate_that_saves_no_input():
    torch.manual_seed(0)
    w = torch.randn(24, 32)
    x = torch.randn(5, 32, requires_grad=True)
    saved = []
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(tuple(t.shape)) or t, lambda t: t):
        y = FrozenLinearFn.apply(x, w, 0)
    assert saved == [(24, 32)]
    g = torch.randn_like(y)
    y.backward(g)
    assert torch.allclose(x.grad, g @ w)
    with pytest.raises(ValueError, match="frozen"):
        FrozenLinearFn.apply(x, w.clone().requires_grad_(), 0)


def test_frozen_coefficients_backward_matches_autograd():
    torch.manual_seed(1)
    mixes = torch.randn(2, 3, 24, requires_grad=True)
    scale, base = torch.full((3,), 0.3), torch.randn(24) * 0.1
    grads = [torch.randn(2, 3, 4), torch.randn(2, 3, 4), torch.randn(2, 3, 4, 4)]
    want, = torch.autograd.grad(hc_split_sinkhorn(mixes, scale, base, 4, 20, 1e-6), mixes, grads)
    got, = torch.autograd.grad(FrozenCoefficientsFn.apply(mixes, scale, base, 4, 20, 1e-6, False), mixes, grads)
    assert torch.allclose(got, want, atol=1e-7)
    carried = FrozenCoefficientsFn.apply(mixes, scale, base, 4, 20, 1e-6, True)
    assert all(v.dtype == torch.float32 and torch.equal(v, v.bfloat16().float()) for v in carried)


@pytest.mark.parametrize("fp8", [False, True])
def test_frozen_backbone_trains_only_what_is_attached(fp8):
    torch.manual_seed(2)
    model = V41LM(V41Config.tiny(fp8=fp8))
    model.init_weights()
    ids = torch.randint(0, 256, (2, 16))
    with torch.no_grad():
        before = model(ids)
    keys = list(model.state_dict())
    receipt = freeze_backbone(model)
    assert list(model.state_dict()) == keys and receipt["trainable_parameters"] == 0 and receipt["expert_sum"] == "fp32, rounded once"
    assert len(receipt["frozen_linears"]) == sum(isinstance(m, QuantLinear) for m in model.modules())
    assert len(receipt["frozen_hyper_connections"]) == sum(isinstance(m, HyperConnectionMix) for m in model.modules()) == 4
    with torch.no_grad():
        after = model(ids)
    assert torch.allclose(after, before, atol=1e-4 if not fp8 else 5e-2)         # weights are rounded once instead of per call
    # a trainable input-side module (stands for an adapter) receives gradients through the frozen stack
    prompt = torch.nn.Parameter(torch.zeros(1, 1, model.config.hidden_size))
    original = model.embed.forward
    model.embed.forward = lambda i: original(i) + prompt
    loss = model(ids, ids)
    loss.backward()
    assert prompt.grad is not None and float(prompt.grad.abs().sum()) > 0
    assert all(p.grad is None for p in model.parameters())
    with pytest.raises(ValueError, match="already frozen"):
        freeze_backbone(model)


@pytest.mark.parametrize("chunk", [1, 3, 128])
def test_frozen_head_cross_entropy_matches_pytorch(chunk):
    from archlab_b200.models.v41_frozen import FrozenHeadCrossEntropy

    torch.manual_seed(3)
    hidden = torch.randn(2, 5, 7, requires_grad=True)
    twin = hidden.detach().clone().requires_grad_()
    weight, labels = torch.randn(23, 7), torch.randint(0, 23, (2, 5))
    labels[:, 1] = -100
    got = FrozenHeadCrossEntropy.apply(hidden, labels, weight, chunk)
    want = torch.nn.functional.cross_entropy((twin @ weight.T).flatten(0, 1), labels.flatten(), reduction="sum")
    (2 * got).backward(), (2 * want).backward()
    assert torch.allclose(got, want, atol=1e-5) and torch.allclose(hidden.grad, twin.grad, atol=1e-5)
    empty = torch.randn(1, 5, 7, requires_grad=True)
    loss = FrozenHeadCrossEntropy.apply(empty, torch.full((1, 5), -100), weight, 3)
    loss.backward()
    assert float(loss.detach()) == 0 and torch.equal(empty.grad, torch.zeros_like(empty))
    with pytest.raises(ValueError, match="frozen"):
        FrozenHeadCrossEntropy.apply(hidden, labels, weight.clone().requires_grad_(), 3)
