"""Pipeline report card: sections, structured summary, wall clock, rank gating."""
import datetime

from archlab_b200.services.run_report import NullReport, RunReport, environment, get_report


def test_card_is_assembled_in_pipeline_order_with_a_summary(tmp_path):
    now = [datetime.datetime(2026, 1, 1, 10, 0, 0)]
    report = RunReport(tmp_path, clock=lambda: now[0])
    report.reset({"commit": "abc1234", "dirty": False, "gpus": {"count": 8}})
    now[0] += datetime.timedelta(hours=2, minutes=5)
    report.log("Chat evaluation sft", [{"ARC-Easy": 0.41234, "GSM8K": 0.05, "ChatCORE": 0.12}, "free text note"])
    now[0] += datetime.timedelta(minutes=10)
    report.log("Base model evaluation", [{"CORE": 0.2213, "tokens": 1234567}, None, {}])
    now[0] += datetime.timedelta(hours=5)
    report.log("Chat evaluation rl", [{"GSM8K": 0.09}])                      # experimental: not part of the wall clock
    text = report.generate().read_text()
    assert text.index("## Base model evaluation") < text.index("## Chat evaluation sft") < text.index("## Summary")
    assert "- tokens: 1,234,567" in text and "- ARC-Easy: 0.4123" in text and "free text note" in text
    rows = [l for l in text.splitlines() if l.startswith("| ") and "Metric" not in l]
    assert rows[0].startswith("| CORE") and rows[-1].startswith("| ChatCORE") and any("GSM8K" in r and "0.0500" in r and "0.0900" in r for r in rows)
    assert "Total wall clock time: 2h15m" in text and "Sections not run: tokenizer-training" in text
    report.reset({"commit": "def"})
    assert not (tmp_path / "base-model-evaluation.md").exists() and not (tmp_path / "report.md").exists()
    assert "Total wall clock time: unknown" in report.generate().read_text()


def test_rank_gating_and_environment(tmp_path):
    assert isinstance(get_report(tmp_path, rank=0), RunReport) and isinstance(get_report(tmp_path, rank=3), NullReport)
    assert get_report(tmp_path, rank=1).log("x", [{"a": 1}]) is None
    env = environment()
    assert {"commit", "dirty", "host", "torch", "gpus"} <= set(env) and env["gpus"]["count"] >= 0
