"""Tied prelude / core / coda execution and Engram geometry scaling (vectors of the reference's
tests/test_prelude_loop_coda.py and tests/test_v41_performance_contract.py)."""
import copy

import pytest
import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from archlab_b200.models.engram_geometry import scaled_engram_geometry
from archlab_b200.models.looped import LoopedStack, LoopLayout, balanced_layout, boundary, loop_blocks


class Block(nn.Module):
    def __init__(self, index):
        super().__init__()
        self.weight = nn.Parameter(torch.randn(4, 4) / 8)
        self.index = index

    def forward(self, hidden, state):
        assert state == self.index          # every core pass re-enters with the carry the prelude handed over
        return checkpoint(lambda x: x + (x @ self.weight).tanh(), hidden, use_reentrant=False), state + 1


@pytest.mark.parametrize("recursions", [1, 2, 4, 12])
def test_tied_forward_and_gradients_match_an_independent_unroll(recursions):
    torch.manual_seed(7)
    blocks = nn.ModuleList(Block(i) for i in range(3))
    oracle = copy.deepcopy(blocks)
    stack = LoopedStack(blocks, LoopLayout(1, 1, 1), repetitions=recursions, step=lambda b, h, s: b(h, s))
    x = torch.randn(2, 3, 2, 4, requires_grad=True)
    xr = x.detach().clone().requires_grad_()
    actual, state = stack(x, 0)
    anchor = xr + (xr @ oracle[0].weight).tanh()
    expected = anchor
    for _ in range(recursions):
        expected = expected + (expected @ oracle[1].weight).tanh()
        expected = expected * (expected.square().mean(-1, keepdim=True) + torch.finfo(torch.float32).eps).rsqrt() + anchor / 2 ** 0.5
    expected = expected + (expected @ oracle[2].weight).tanh()
    torch.testing.assert_close(actual, expected, rtol=1e-6, atol=1e-6)
    actual.square().sum().backward()
    expected.square().sum().backward()
    torch.testing.assert_close(x.grad, xr.grad, rtol=1e-5, atol=2e-5)
    for p, q in zip(blocks.parameters(), oracle.parameters(), strict=True):
        torch.testing.assert_close(p.grad, q.grad, rtol=1e-5, atol=2e-5)
    assert stack.visits == [1, recursions, 1] and state == 3
    assert len(list(stack.state_dict())) == 3           # tied blocks are stored once


def test_two_live_graphs_keep_their_own_anchor():
    torch.manual_seed(0)
    stack = LoopedStack([nn.Linear(4, 4) for _ in range(3)], LoopLayout(1, 1, 1))
    x, y = torch.randn(2, 4, requires_grad=True), torch.randn(2, 4, requires_grad=True)
    a, b = stack(x), stack(y)
    (a.sum() + 0 * b.sum()).backward()
    assert x.grad.abs().sum() > 0 and y.grad.abs().sum() == 0


def test_layout_rules():
    assert LoopLayout().stored_depth == 20 and LoopLayout(2, 3, 1).execution(2) == [0, 1, 2, 3, 4, 2, 3, 4, 5]
    assert [balanced_layout(d) for d in (9, 10, 11)] == [LoopLayout(3, 3, 3), LoopLayout(3, 4, 3), LoopLayout(3, 4, 4)]
    for bad in (dict(prelude=0), dict(core=True), dict(coda=-1)):
        with pytest.raises(ValueError):
            LoopLayout(**bad)
    with pytest.raises(ValueError):
        LoopLayout().execution(0)
    h, a = torch.randn(3, 8), torch.randn(3, 8)
    torch.testing.assert_close(boundary(h, a), h * (h.square().mean(-1, keepdim=True) + torch.finfo(torch.float32).eps).rsqrt() + a / 2 ** 0.5)
    model = nn.Module()
    model.layers = nn.ModuleList(nn.Linear(4, 4) for _ in range(7))
    stack = loop_blocks(model, "layers", repetitions=3)
    assert stack.layout == LoopLayout(2, 3, 2) and model.layers(torch.randn(2, 4)).shape == (2, 4) and stack.visits == [1, 1, 3, 3, 3, 1, 1]


BASE = dict(hidden_size=5120, engram_head_dim=256, engram_vocab_size=16_000_000, engram_layer_ids=[1, 14],
            engram_max_ngram_size=4, engram_n_heads=8)


def test_engram_geometry_scales_buckets_and_aligns_channels():
    g = scaled_engram_geometry(BASE, 128)
    assert g["engram_head_dim"] == 8 and g["engram_vocab_size"] == 400_000
    assert all(9_600_000 < rows < 9_620_000 for rows in g["engram_num_embeddings"])
    assert g["engram_num_embeddings"][0] != g["engram_num_embeddings"][1]
    assert scaled_engram_geometry(BASE, 640)["engram_head_dim"] == 32
    assert scaled_engram_geometry(BASE, 640)["engram_vocab_size"] == 2_000_000


def test_fixed_lookup_budget_is_independent_of_width():
    anchor = scaled_engram_geometry(BASE, 128)
    for width in (128, 256, 384, 640, 1280):
        assert scaled_engram_geometry(BASE, width, anchor_width=128) == anchor
    with pytest.raises(ValueError):
        scaled_engram_geometry(BASE, 128, anchor_width=0)
    # the primes of one (layer, order) ascend head by head from the bucket count, and no prime is used twice
    small = dict(hidden_size=8, engram_head_dim=8, engram_vocab_size=10, engram_layer_ids=[0], engram_max_ngram_size=3, engram_n_heads=2)
    assert scaled_engram_geometry(small, 8)["engram_num_embeddings"] == [11 + 13 + 17 + 19]
