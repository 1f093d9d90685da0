"""Order-fixed fp32 sums: values, gradients, input validation, order sensitivity that the fixed order removes."""
import pytest
import torch

from archlab_b200.ops.ordered import ordered_index_sum, ordered_permutation_sum


def test_index_sum_adds_in_input_order_with_one_write_per_row():
    dest = torch.zeros(4, 2)
    idx = torch.tensor([2, 0, 2, 2, 3])
    vals = torch.tensor([[1e8, 1.0], [5.0, 5.0], [1.0, 1.0], [-1e8, 2.0], [7.0, 7.0]])
    ordered_index_sum(dest, idx, vals)
    assert dest[0].tolist() == [5.0, 5.0] and dest[3].tolist() == [7.0, 7.0] and dest[1].tolist() == [0.0, 0.0]
    assert dest[2].tolist() == [float((torch.tensor(1e8) + 1.0) - 1e8), 4.0]          # (1e8 + 1) - 1e8 in fp32, not 1e8 - 1e8 + 1
    assert ordered_index_sum(torch.ones(2, 2), torch.zeros(0, dtype=torch.long), torch.zeros(0, 2)).tolist() == [[1, 1], [1, 1]]


def test_permutation_sum_matches_the_definition_and_its_backward_is_a_permutation():
    torch.manual_seed(0)
    tokens, slots, width = 37, 3, 5
    counts = torch.randint(1, slots + 1, (tokens,))
    positions = torch.full((tokens, slots), -1, dtype=torch.long)
    perm = torch.randperm(int(counts.sum()))
    at = 0
    for t in range(tokens):
        positions[t, :counts[t]] = perm[at:at + counts[t]]
        at += int(counts[t])
    values = torch.randn(int(counts.sum()), width, dtype=torch.bfloat16, requires_grad=True)
    out = ordered_permutation_sum(values, positions, chunk_rows=8)
    want = torch.stack([sum((values[p].float() for p in positions[t] if p >= 0), torch.zeros(width)) for t in range(tokens)])
    assert out.dtype == torch.float32 and torch.equal(out, want)
    g = torch.randn_like(out)
    out.backward(g)
    for t in range(tokens):
        for p in positions[t]:
            if p >= 0:
                assert torch.equal(values.grad[p], g[t].bfloat16())
    again = ordered_permutation_sum(values.detach(), positions, chunk_rows=1000)
    assert torch.equal(again, out.detach())                                            # chunking does not change a bit


def test_validation():
    v = torch.randn(3, 2)
    with pytest.raises(ValueError, match="permutation"):
        ordered_permutation_sum(v, torch.tensor([[0, 1], [1, -1]]))                    # row 1 twice, row 2 never
    with pytest.raises(ValueError, match="permutation"):
        ordered_permutation_sum(v, torch.tensor([[0, 1], [2, -2]]))
    with pytest.raises(ValueError, match="floating rows"):
        ordered_permutation_sum(v.long(), torch.tensor([[0, 1], [2, -1]]))
    with pytest.raises(ValueError, match="chunk size"):
        ordered_permutation_sum(v, torch.tensor([[0, 1], [2, -1]]), chunk_rows=0)
    assert ordered_permutation_sum(v, torch.tensor([[2, 0], [1, -1]])).shape == (2, 2)
