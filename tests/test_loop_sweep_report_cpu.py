"""Sweep report: contract-checked measurements, compute-matched cuts, convex envelope, tuned weight decay."""
import json
import math

import pytest

from archlab_b200.services import loop_sweep_report as rp
from archlab_b200.train import loop_sweep as ls


def test_interpolation_never_extrapolates_and_the_envelope_is_convex():
    pts = [{"compute": 10.0, "loss": 3.0}, {"compute": 100.0, "loss": 2.0}]
    assert rp.interpolate(pts, 55.0) == pytest.approx(2.5) and rp.interpolate(pts, 100.0) == 2.0
    assert rp.interpolate(pts, 5.0) is None and rp.interpolate(pts, 500.0) is None
    cloud = [{"compute": 10.0, "loss": 3.0}, {"compute": 31.6, "loss": 2.9}, {"compute": 100.0, "loss": 2.0}, {"compute": 300.0, "loss": 2.1},
             {"compute": 1000.0, "loss": 1.8}, {"compute": 20.0, "loss": 3.5}]
    hull = rp.envelope(cloud)
    assert [p["compute"] for p in hull] == [10.0, 100.0, 1000.0]                   # 31.6 lies above the chord, 300 and 20 are dominated


def synthetic(plan_dir, finished):
    base = {"root": str(plan_dir / "campaign"), "environment": {"PYTHONPATH": "/src"}, "runs": [{"variant": "normal", "width": 128}]}
    (plan_dir / "base.json").write_text(json.dumps(base))
    plan = ls.write_plan(plan_dir / "base.json", source=plan_dir / "checkout", commit="abc", destination=plan_dir / "plan.json")
    for run in plan["runs"]:
        c = run["cell"]
        if not finished(c):
            continue
        out = plan_dir / "campaign" / ls.cell_name(c)
        out.mkdir(parents=True)
        compute = 100.0 * c["stored_layers"] * c["recursions"] * (c["hidden_size"] / 128) ** 2
        loss = 4.0 - 0.35 * math.log10(compute) + 0.2 * abs(c["weight_decay"] - (0.8 if c["recursions"] > 1 else 0.4))
        rows = [{"step": 0, "loss": 9.0, "consumed_supervised_tokens": 0, "training_gpu_seconds": 0.0},
                {"step": 50, "loss": loss + 0.5, "consumed_supervised_tokens": 5 * 10 ** 8, "training_gpu_seconds": compute / 2},
                {"step": 100, "loss": loss, "consumed_supervised_tokens": 10 ** 9, "training_gpu_seconds": compute}]
        (out / "validation.jsonl").write_text("".join(json.dumps(r) + "\n" for r in rows))
        (out / "COMPLETE.json").write_text(json.dumps({"passed": True, "supervised_tokens": 10 ** 9, "step": 100, "training_gpu_seconds": compute}))
        (out / "RUN_CONTRACT.json").write_text(json.dumps({"repeated_data_sweep": c, "project_commit": "abc"}))
    return plan


def test_report_over_the_registered_grid(tmp_path):
    plan = synthetic(tmp_path, lambda c: c["reference_depth"] in (6, 8, 10))
    summary = rp.report(tmp_path / "plan.json", tmp_path / "report")
    n = sum(len(ls.GRID[d]) for d in (6, 8, 10)) * 6
    assert summary["registered_cells"] == 222 and summary["completed_cells"] == n and summary["trajectory_points"] == 2 * n
    analysis = summary["analysis"]
    assert len(analysis["cuts"]) >= 5 and all(len(c["losses"]) >= 2 for c in analysis["cuts"])
    wd = {(r["reference_depth"], r["recursions"]): r["weight_decay"] for r in analysis["optimal_weight_decay"]}
    assert wd[(8, 1)] == 0.4 and wd[(8, 2)] == 0.8 and len(wd) == n // 6
    k1 = analysis["recipes"]["K1, fixed weight decay"]
    assert [p["reference_depth"] for p in k1] == [6, 8, 10]
    front = analysis["recipes"]["loop frontier, fixed weight decay"]
    assert front and front[-1]["compute"] <= max(p["compute"] for p in front) and all(a["loss"] > b["loss"] for a, b in zip(front, front[1:]))
    assert (tmp_path / "report" / "final.csv").read_text().count("\n") == n + 1
    broken = tmp_path / "campaign" / "loop-d128-L20-K2-wd0p8" / "COMPLETE.json"
    broken.write_text(json.dumps({**json.loads(broken.read_text()), "supervised_tokens": 999}))
    with pytest.raises(ValueError, match="registered contract"):
        rp.report(tmp_path / "plan.json", tmp_path / "report2")
    plan["runs"].pop()
    with pytest.raises(ValueError, match="preregistered grid"):
        rp.load_measurements(plan)
