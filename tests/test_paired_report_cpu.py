"""Token-matched paired report from two training ledgers."""
import csv
import json

import pytest

from archlab_b200.services import reporting as rp


def _ledger(directory, losses, *, first_step=1, tokens=100, lr=1e-3, history=None, torn=False):
    directory.mkdir(parents=True, exist_ok=True)
    rows = [{"step": first_step + i, "loss": l, "supervised_tokens": tokens, "consumed_supervised_tokens": tokens * (first_step + i),
             "learning_rate": lr} for i, l in enumerate(losses)]
    body = "".join(json.dumps(r) + "\n" for r in rows) + ('{"step": 99, "lo' if torn else "")
    (directory / "train-metrics.jsonl").write_text(body)
    if history:
        (directory / "prior-phase-metrics.jsonl").write_text("".join(json.dumps(r) + "\n" for r in history))
    return rows


def test_ledger_validation_and_windows(tmp_path):
    _ledger(tmp_path / "a", [4.0, 3.0, 2.0, 1.0], torn=True)
    led = rp.TrainingLedger.read(tmp_path / "a")
    assert len(led.rows) == 4 and led.token_interval == (0, 400) and led.sources[0]["rows"] == 4
    assert led.window_mean(0, 400) == pytest.approx(2.5) and led.window_mean(150, 350) == pytest.approx((50 * 3 + 100 * 2 + 50 * 1) / 200)
    assert led.smoothed(200)[-1] == (400, pytest.approx(1.5))
    bad = [dict(r) for r in led.rows]
    bad[2]["step"] = 7
    with pytest.raises(ValueError, match="non-contiguous"):
        rp.TrainingLedger(bad)
    bad = [dict(r) for r in led.rows]
    bad[1]["consumed_supervised_tokens"] += 1
    with pytest.raises(ValueError, match="cumulative cursor"):
        rp.TrainingLedger(bad)
    with pytest.raises(json.JSONDecodeError):
        rp.TrainingLedger.decode(b'{"a": 1}\n{broken\n{"a": 2}\n')
    with pytest.raises(ValueError, match="empty token window"):
        led.window_mean(1000, 2000)


def test_paired_report_matches_updates_and_refuses_different_cursors(tmp_path):
    hist = [{"step": 1, "loss": 9.0, "supervised_tokens": 100, "consumed_supervised_tokens": 100, "learning_rate": 1e-3}]
    _ledger(tmp_path / "base", [4.0, 3.0, 2.0, 1.0], first_step=2, history=hist)
    _ledger(tmp_path / "arm", [4.5, 2.5, 1.5], first_step=2, history=hist)
    out = rp.paired_report({"base": str(tmp_path / "base"), "arm": str(tmp_path / "arm")}, tmp_path / "report", smoothing_tokens=200,
                           summary_tokens=200)
    assert out["matched_steps"] == [1, 4] and out["matched_token_interval"] == [0, 400] and out["summary_token_interval"] == [200, 400]
    assert out["runs"]["base"]["matched_token_weighted_ce"] == pytest.approx(2.5) and out["runs"]["arm"]["matched_token_weighted_ce"] == pytest.approx(2.0)
    assert out["first_minus_second_ce"] == pytest.approx(0.5) and out["runs"]["base"]["latest_step"] == 5
    rows = list(csv.reader(open(tmp_path / "report" / "matched-training-curves.csv")))
    assert rows[0][:4] == ["step", "supervised_tokens", "base", "arm"] and len(rows) == 5 and float(rows[-1][4]) == pytest.approx(2.5)
    assert json.loads((tmp_path / "report" / "SUMMARY.json").read_text())["smoothing_tokens"] == 200
    with pytest.raises(FileExistsError):
        rp.paired_report({"base": str(tmp_path / "base"), "arm": str(tmp_path / "arm")}, tmp_path / "report")
    only_current = rp.paired_report({"base": str(tmp_path / "base"), "arm": str(tmp_path / "arm")}, tmp_path / "r2", current_phase_only=True,
                                    smoothing_tokens=100, summary_tokens=1000)
    assert only_current["matched_steps"] == [2, 4]
    _ledger(tmp_path / "other_lr", [4.0, 3.0], first_step=2, lr=5e-4)
    with pytest.raises(ValueError, match="paired learning_rate differs"):
        rp.paired_report({"base": str(tmp_path / "base"), "x": str(tmp_path / "other_lr")}, tmp_path / "r3", current_phase_only=True)
    assert rp.main(["--run", "base", str(tmp_path / "base"), "--run", "arm", str(tmp_path / "arm"), "--output", str(tmp_path / "r4")]) == 0


def test_runs_with_different_batch_sizes_share_a_token_axis():
    import pytest

    from archlab_b200.services.reporting import aligned_curves, token_blocks, trailing_means

    small = [{"step": s, "loss": 4.0 - 0.01 * s} for s in range(1, 41)]                     # 100 tokens per step
    large = [{"step": s, "loss": 3.9 - 0.04 * s} for s in range(1, 11) if s != 7]           # 400 tokens per step, step 7 lost
    a = token_blocks(small, tokens_per_step=100, block_tokens=800)
    assert [p["tokens"] for p in a] == [800, 1600, 2400, 3200, 4000] and a[0]["loss"] == pytest.approx(4.0 - 0.01 * 4.5)
    b = token_blocks(large, tokens_per_step=400, block_tokens=800)
    assert [p["block"] for p in b] == [1, 2, 3, 5]                                            # block 4 (steps 7-8) is incomplete and left out
    with pytest.raises(ValueError, match="whole number"):
        token_blocks(small, tokens_per_step=300, block_tokens=800)
    with pytest.raises(ValueError, match="no complete"):
        token_blocks(small[:3], tokens_per_step=100, block_tokens=800)
    assert trailing_means([1.0, 3.0, 5.0, 7.0], 2) == [1.0, 2.0, 4.0, 6.0]
    out = aligned_curves({"small": (small, 100), "large": (large, 400)}, block_tokens=800, smoothing_blocks=2)
    deltas = out["differences"]["large"]
    assert [d["tokens"] for d in deltas] == [800, 1600, 2400, 4000] and all(d["delta"] < 0 for d in deltas) and out["differences_against"] == "small"
