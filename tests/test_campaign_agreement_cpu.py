"""Campaign aggregation: contract validation, overlays vs recoveries, same-seed pairing, cross-backend agreement."""
import dataclasses
import json

import pytest

from archlab_b200.contracts.campaigns import TEN_M_SEEDS, TEN_M_VARIANTS_BY_NAME
from archlab_b200.services import campaign_agreement as cc


def row(backend, variant, seed, bpb, tps, steady=None):
    c = TEN_M_VARIANTS_BY_NAME[variant]
    return cc.RunResult(backend, variant, seed, c.parameter_count, c.steps, c.training_tokens, bpb, tps, 100.0, steady_state_tokens_per_second=steady)


def campaign(backend, shift=0.0, speed=1000.0):
    rows = []
    for i, v in enumerate(TEN_M_VARIANTS_BY_NAME):
        for s in TEN_M_SEEDS:
            effect = 0.0 if v == "baseline" else (-0.01 if i % 2 else 0.005) * (1 + shift)
            rows.append(row(backend, v, s, 1.5 + 0.001 * s + effect, speed * (1 - 0.01 * i)))
    return rows


def test_pairing_and_cross_backend_agreement(tmp_path):
    rows = cc.validate(campaign("speedrun") + campaign("mesh", shift=0.2, speed=3000.0))
    summaries = cc.summarize(rows)
    gdn = next(s for s in summaries if s["backend"] == "speedrun" and s["variant"] == "qwen-gdn")
    assert gdn["seeds"] == len(TEN_M_SEEDS) and gdn["paired_delta_bpb"] == pytest.approx(-0.01) and gdn["throughput_basis"] == "aggregate after warm-up"
    metrics = cc.write_comparison(tmp_path / "out", rows, "speedrun", "mesh")
    assert metrics["variant_count"] == 15 and metrics["delta_pearson"] == pytest.approx(1.0) and metrics["delta_sign_agreement_rate"] == 1.0
    assert metrics["baseline_absolute_throughput_ratio"] == pytest.approx(3.0) and metrics["baseline_bpb_gap"] == pytest.approx(0.0)
    assert (tmp_path / "out" / "comparison.md").read_text().count("\n| ") >= 16
    assert json.loads((tmp_path / "out" / "comparison.json").read_text())["metrics"]["variant_count"] == 15
    assert len(cc.load_table(tmp_path / "out" / "runs.csv")) == len(rows)
    steady = [dataclasses.replace(r, steady_state_tokens_per_second=2 * r.tokens_per_second) for r in campaign("speedrun")]
    assert cc.summarize(steady)[0]["throughput_basis"] == "median steady-state step"


def test_contract_and_completeness(tmp_path):
    rows = campaign("speedrun")
    with pytest.raises(ValueError, match="missing 1 frozen runs"):
        cc.validate(rows[:-1])
    assert len(cc.validate(rows[:-1], allow_partial=True)) == len(rows) - 1
    with pytest.raises(ValueError, match="contract drift"):
        cc.validate([dataclasses.replace(rows[0], training_steps=1)], allow_partial=True)
    with pytest.raises(ValueError, match="invalid final_bpb"):
        cc.validate([dataclasses.replace(rows[0], final_bpb=float("nan"))], allow_partial=True)
    with pytest.raises(ValueError, match="unexpected campaign row"):
        cc.validate([dataclasses.replace(rows[0], seed=999)], allow_partial=True)
    with pytest.raises(ValueError, match="duplicate"):
        cc.validate(rows + rows[:1])
    fixed = cc.overlay(rows, [dataclasses.replace(rows[3], final_bpb=1.0)])
    assert len(fixed) == len(rows) and min(r.final_bpb for r in fixed) == 1.0
    with pytest.raises(ValueError, match="unknown rows"):
        cc.overlay(rows[1:], rows[:1])
    assert len(cc.merge_recoveries(rows[1:], rows[:1])) == len(rows)
    with pytest.raises(ValueError, match="would replace"):
        cc.merge_recoveries(rows, rows[:1])
    run_dir = tmp_path / "results" / "baseline-s0"
    run_dir.mkdir(parents=True)
    r = rows[0]
    (run_dir / "result.json").write_text(json.dumps({"backend": "mesh", "mode": "full", "variant": {"name": r.variant}, "seed": r.seed, "parameter_count": r.parameter_count,
                                                       "training_steps": r.training_steps, "training_tokens": r.training_tokens, "final_bpb": 1.4, "tokens_per_second": 10.0,
                                                       "wall_seconds": 5.0, "optimization_recipe": {"name": "baseline"}}))
    loaded = cc.load_results(tmp_path / "results", "mesh")
    assert len(loaded) == 1 and loaded[0].variant == r.variant and loaded[0].optimization_recipe == "baseline" and cc.load_results(tmp_path / "results", "speedrun") == []
