"""Per-token loss normalisation: uneven micro-batches give the gradient of the global token mean."""
import pytest
import torch

from archlab_b200.train.token_loss import TokenNormalizedStep, component_mean_loss, masked_token_loss


def test_uneven_micro_batches_equal_the_global_token_mean():
    torch.manual_seed(0)
    w = torch.nn.Parameter(torch.randn(5, 7))
    x = torch.randn(3, 6, 5)
    labels = torch.randint(0, 7, (3, 6))
    labels[0, 1:] = -1                                               # micro-batch 0 supervises a single token
    labels[2, 4:] = -1

    def losses(i):
        return torch.nn.functional.cross_entropy((x[i] @ w), labels[i].clamp_min(0), reduction="none")

    mask = labels.ne(-1)
    reference = sum((losses(i) * mask[i]).sum() for i in range(3)) / mask.sum()
    (g_ref,) = torch.autograd.grad(reference, w)
    step = TokenNormalizedStep()
    for i in range(3):
        total, count, report = masked_token_loss(mask[i], losses(i))
        assert int(report["lm loss"][1]) == int(mask[i].sum())
        step.backward(total, count)
    out = step.finish([w])
    assert out["global_tokens"] == int(mask.sum()) and out["loss"] == pytest.approx(float(reference.detach()), rel=1e-6)
    assert torch.allclose(w.grad, g_ref, atol=1e-6)
    w.grad = None
    naive = sum((losses(i) * mask[i]).sum() / mask[i].sum() for i in range(3)) / 3          # mean of micro-batch means: a different objective
    (g_naive,) = torch.autograd.grad(naive, w)
    assert not torch.allclose(g_naive, g_ref, atol=1e-4)
    with pytest.raises(RuntimeError, match="no micro-batch"):
        step.finish([w])


def test_auxiliary_sums_share_the_denominator_and_legacy_mean():
    w = torch.nn.Parameter(torch.ones(3))
    step = TokenNormalizedStep()
    step.backward((w * torch.tensor([1.0, 2.0, 3.0])).sum(), torch.tensor(4), 0.5 * (w ** 2).sum())
    out = step.finish([w], gradients_are_averaged=False)
    assert out["gradient_scale"] == 0.25 and torch.allclose(w.grad, (torch.tensor([1.0, 2.0, 3.0]) + 1.0) / 4)
    loss, report = component_mean_loss(torch.tensor([[1.0, 3.0]]), {"aux": torch.tensor(0.5)})
    assert float(loss) == 2.0 and report["lm loss"].tolist() == [4.0, 2.0] and report["aux"].tolist() == [0.5, 1.0]
    step.backward(torch.zeros((), requires_grad=True) * 1.0, torch.tensor(0))
    with pytest.raises(RuntimeError, match="no supervised token"):
        step.finish([w])
