"""Gradient admission: exactness where it is owed, noise-derived bounds elsewhere, and controls that can say no."""
import json

import pytest
import torch

from archlab_b200.train.gradient_oracle import collect_gradients, gradient_admission, pair_metrics


def grads(scale=1.0, noise=0.0, seed=0):
    g = torch.Generator().manual_seed(1)
    base = {"a.weight": torch.randn(8, 8, generator=g), "b.weight": torch.randn(4, generator=g)}
    n = torch.Generator().manual_seed(100 + seed)
    return {k: v * scale + noise * torch.randn(v.shape, generator=n) for k, v in base.items()}


def noisy_reference(level):
    calls = [0]

    def run():
        calls[0] += 1
        return grads(noise=level, seed=calls[0])
    return run


def test_bounded_native_variation_is_allowed(tmp_path):
    report = gradient_admission(grads(noise=1e-4, seed=9), noisy_reference(1e-4), atomic=True, report_path=tmp_path / "oracle.json")
    assert len(report["unchanged_native_controls"]) == 2 and report["bridge"]["global_relative"] <= report["bound"]
    assert json.loads((tmp_path / "oracle.json").read_text())["native_noise"] > 0


def test_deterministic_paths_must_be_bit_exact():
    assert gradient_admission(grads(), lambda: grads(), atomic=False)["bound"] == 0.0
    with pytest.raises(AssertionError, match="bit-exact"):
        gradient_admission(grads(scale=1.000001), lambda: grads(), atomic=False)


def test_scaled_gradients_fail_globally_and_unstable_controls_block_admission(tmp_path):
    with pytest.raises(AssertionError, match="global gradient error"):
        gradient_admission(grads(scale=1.1), noisy_reference(1e-4), atomic=True, report_path=tmp_path / "scaled.json")
    assert json.loads((tmp_path / "scaled.json").read_text())["bridge"]["norm_ratio"] == pytest.approx(1.1, rel=1e-3)   # written even on failure
    with pytest.raises(AssertionError, match="native control exceeds"):
        gradient_admission(grads(), noisy_reference(0.5), atomic=True)
    wrong = grads()
    wrong["b.weight"] = wrong["b.weight"] + 0.004                      # small tensor: invisible globally at a loose bound, caught per tensor
    with pytest.raises(AssertionError, match="per-tensor"):
        gradient_admission(wrong, noisy_reference(2e-4), atomic=True, margin=8.0, per_tensor_factor=1.5)
    with pytest.raises(AssertionError, match="gradient sets differ"):
        pair_metrics({"a.weight": torch.ones(1)}, {"c.weight": torch.ones(1)})


def test_gradients_are_read_from_where_the_backward_put_them():
    m = torch.nn.Linear(2, 2)
    m.weight.main_grad, m.weight.grad_added_to_main_grad = torch.full((2, 2), 3.0), True
    m.bias.grad = torch.ones(2)
    got = collect_gradients(m)
    assert torch.equal(got["weight"], torch.full((2, 2), 3.0)) and torch.equal(got["bias"], torch.ones(2))
