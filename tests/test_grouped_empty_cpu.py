"""A rank that receives no expert rows must still run the backward of whatever produced its (empty) input: expert dispatch
is an autograd function with barriers inside, and a rank that skips it leaves its peers waiting."""
import torch

from archlab_b200.ops import grouped


def test_empty_grouped_input_keeps_its_producer_in_the_graph():
    seen = []

    class Producer(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x):
            return x[:0].clone()

        @staticmethod
        def backward(ctx, g):
            seen.append(tuple(g.shape))
            return torch.zeros(4, 3)

    x = torch.randn(4, 3, requires_grad=True)
    w = torch.randn(2, 5, 3, requires_grad=True)
    h = grouped.grouped_linear(Producer.apply(x), w, torch.zeros(0, dtype=torch.int32), [0, 0], [0, 0])
    assert h.shape == (0, 5)
    h.sum().backward()
    assert seen == [(0, 3)] and float(w.grad.abs().sum()) == 0.0 and x.grad is not None
