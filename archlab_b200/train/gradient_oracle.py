"""Admitting a new backward path by its gradients, with negative controls that make the verdict mean something.

A candidate implementation (a fused kernel path, a sharded execution) is compared with a reference implementation on the
same batch.  How close is close enough depends on whether the REFERENCE itself is reproducible:

* ``atomic=False`` (no atomics or unordered reductions anywhere): the candidate must be bit-exact.  A tolerance here
  would hide indexing errors on tiny fixtures.
* ``atomic=True``: the reference is run ``controls`` more times on the same inputs.  The spread between those
  unchanged native runs is the noise floor; if it already exceeds ``max_native_relative`` the fixture is too unstable to
  admit anything and the oracle says so.  The candidate passes when its GLOBAL relative error (all tensors as one
  vector) is within ``max(noise x margin, floor)`` and no single tensor is off by more than ``per_tensor_factor`` times
  that bound -- a uniformly scaled gradient (a wrong loss normalisation) fails the global test even though every element
  looks "close".
The report lists per-tensor metrics, the controls and the bounds used, and is written next to the run's evidence.
(Reference: the admission helpers of tests/integration/test_megatron_agentic_training.py as exercised by
tests/test_training_gradient_oracle.py:31-70.)
"""
from __future__ import annotations

import json
from pathlib import Path
from typing import Callable

import torch


def _flat(grads: dict[str, torch.Tensor]) -> torch.Tensor:
    return torch.cat([grads[k].detach().double().flatten() for k in sorted(grads)])


def pair_metrics(actual: dict[str, torch.Tensor], expected: dict[str, torch.Tensor]) -> dict:
    if actual.keys() != expected.keys():
        raise AssertionError(f"gradient sets differ: {sorted(actual.keys() ^ expected.keys())[:5]}")
    a, e = _flat(actual), _flat(expected)
    per_tensor = {}
    for name in sorted(actual):
        x, y = actual[name].detach().double(), expected[name].detach().double()
        per_tensor[name] = {"relative": float((x - y).norm() / y.norm().clamp_min(1e-30)), "max_abs": float((x - y).abs().max()),
                            "bit_exact": bool(torch.equal(actual[name], expected[name]))}
    return {"global_relative": float((a - e).norm() / e.norm().clamp_min(1e-30)), "cosine": float(torch.dot(a, e) / (a.norm() * e.norm()).clamp_min(1e-30)),
            "norm_ratio": float(a.norm() / e.norm().clamp_min(1e-30)), "bit_exact": all(t["bit_exact"] for t in per_tensor.values()), "per_tensor": per_tensor}


def gradient_admission(candidate: dict[str, torch.Tensor], reference: Callable[[], dict[str, torch.Tensor]], *, atomic: bool, controls: int = 2,
                       margin: float = 4.0, floor: float = 1e-6, max_native_relative: float = 1e-2, per_tensor_factor: float = 8.0,
                       report_path=None) -> dict:
    expected = reference()
    report = {"atomic": atomic, "bridge": pair_metrics(candidate, expected), "unchanged_native_controls": []}
    try:
        if not atomic:
            if not report["bridge"]["bit_exact"]:
                worst = max(report["bridge"]["per_tensor"].items(), key=lambda kv: kv[1]["max_abs"])
                raise AssertionError(f"a deterministic path must be bit-exact; {worst[0]} differs by {worst[1]['max_abs']:.3e}")
            report["bound"] = 0.0
            return report
        noise = 0.0
        for _ in range(controls):
            control = pair_metrics(reference(), expected)
            report["unchanged_native_controls"].append({"global_relative": control["global_relative"]})
            noise = max(noise, control["global_relative"])
        if noise > max_native_relative:
            raise AssertionError(f"native control exceeds the admissible variation ({noise:.3e} > {max_native_relative:.1e}); the fixture cannot admit anything")
        bound = max(noise * margin, floor)
        report["bound"], report["native_noise"] = bound, noise
        if report["bridge"]["global_relative"] > bound:
            raise AssertionError(f"global gradient error {report['bridge']['global_relative']:.3e} exceeds {bound:.3e} "
                                 f"(norm ratio {report['bridge']['norm_ratio']:.6f})")
        bad = {n: t["relative"] for n, t in report["bridge"]["per_tensor"].items() if t["relative"] > per_tensor_factor * bound}
        if bad:
            raise AssertionError(f"per-tensor gradient error exceeds {per_tensor_factor * bound:.3e}: {sorted(bad.items(), key=lambda kv: -kv[1])[:3]}")
        return report
    finally:
        if report_path is not None:
            Path(report_path).parent.mkdir(parents=True, exist_ok=True)
            Path(report_path).write_text(json.dumps(report, indent=1) + "\n")


def collect_gradients(model: torch.nn.Module) -> dict[str, torch.Tensor]:
    """``.main_grad`` where a fused accumulation wrote there, ``.grad`` otherwise."""
    out = {}
    for name, p in model.named_parameters():
        g = p.main_grad if getattr(p, "grad_added_to_main_grad", False) or (p.grad is None and hasattr(p, "main_grad")) else p.grad
        if g is not None:
            out[name] = g.detach().clone()
    return out
