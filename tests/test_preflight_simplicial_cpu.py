"""Simplicial kernel preflight as a runnable gate: ladder + causality + receipt, and a failing case stops it."""
import json

import pytest
import torch

from archlab_b200.train import preflight_simplicial as P


def test_ladder_passes_on_the_pytorch_statement_and_writes_a_receipt(tmp_path):
    out = tmp_path / "receipt.json"
    ev = P.run(out, device="cpu", ladder=((1, 1, 1), (17, 3, 8), (35, 16, 32)))
    saved = json.loads(out.read_text())
    assert saved["status"] == ev["status"] == "passed" and len(saved["correctness"]) == 3 and saved["benchmarks"] == []
    case = saved["correctness"][1]
    assert case["future_perturbation_exact"] and case["gradients_finite"] and set(case["errors"]) == {"output", "dq", "dk1", "dk2", "dv1", "dv2"}
    assert all(e["relative_l2"] <= 1e-4 for e in case["errors"].values())
    assert "ops/simplicial.py" in saved["source_sha256"] and saved["training_started"] is False
    with pytest.raises(ValueError, match="refusing to overwrite"):
        P.run(out, device="cpu", ladder=((1, 1, 1),))


def test_a_failing_case_ends_the_gate_with_the_evidence_so_far(tmp_path, monkeypatch):
    real = P.simplicial_attention
    monkeypatch.setattr(P, "simplicial_attention", lambda *a, **k: real(*a, **k) * 1.01)       # a wrong kernel
    out = tmp_path / "receipt.json"
    with pytest.raises(RuntimeError, match="numerical gate failed"):
        P.run(out, device="cpu", ladder=((17, 3, 8), (35, 16, 32)))
    saved = json.loads(out.read_text())
    assert saved["status"] == "failed" and len(saved["correctness"]) == 1 and not saved["correctness"][0]["passed"]
