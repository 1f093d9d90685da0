"""Chunked trainable-head cross entropy equals PyTorch's in value and in both gradients, and keeps no logits."""
import pytest
import torch

from archlab_b200.ops.chunked_ce import ChunkedHeadCrossEntropy, chunked_head_cross_entropy


@pytest.mark.parametrize("chunk", [1, 4, 1000])
def test_values_and_gradients(chunk):
    torch.manual_seed(0)
    h = torch.randn(2, 7, 6, requires_grad=True)
    w = torch.randn(19, 6, requires_grad=True)
    h2, w2 = h.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    labels = torch.randint(0, 19, (2, 7))
    labels[0, :3] = -100
    got = chunked_head_cross_entropy(h, labels, w, chunk_tokens=chunk)
    want = torch.nn.functional.cross_entropy((h2 @ w2.T).flatten(0, 1), labels.flatten(), ignore_index=-100)
    (3 * got).backward(), (3 * want).backward()
    assert torch.allclose(got, want, atol=1e-6) and torch.allclose(h.grad, h2.grad, atol=1e-6) and torch.allclose(w.grad, w2.grad, atol=1e-6)
    assert torch.equal(h.grad[0, :3], torch.zeros(3, 6))


def test_nothing_vocabulary_sized_is_saved_and_inputs_are_checked():
    h, w = torch.randn(3, 5, 4, requires_grad=True), torch.randn(50, 4, requires_grad=True)
    labels = torch.randint(0, 50, (3, 5))
    saved = []
    with torch.autograd.graph.saved_tensors_hooks(lambda t: saved.append(t.numel()) or t, lambda t: t):
        loss = ChunkedHeadCrossEntropy.apply(h, labels, w, 4)
    assert sorted(saved) == sorted([h.numel(), labels.numel(), w.numel()])
    loss.backward()
    frozen = chunked_head_cross_entropy(h.detach().requires_grad_(), labels, w.detach(), reduction="sum")
    frozen.backward()
    empty = chunked_head_cross_entropy(h, torch.full((3, 5), -100), w)
    empty.backward()
    assert float(empty.detach()) == 0
    with pytest.raises(ValueError, match="shapes"):
        chunked_head_cross_entropy(h, labels[:, :4], w)
    with pytest.raises(ValueError, match="positive integer"):
        chunked_head_cross_entropy(h, labels, w, chunk_tokens=0)
    with pytest.raises(ValueError, match="reduction"):
        chunked_head_cross_entropy(h, labels, w, reduction="none")
