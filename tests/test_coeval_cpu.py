"""Evaluation beside training: ledger tails, yield rules, own-children-only signalling."""
import json
import sys
import time

import pytest

from archlab_b200.services import coeval


def ledger(root, n=5, seconds=2.0):
    root.mkdir(parents=True, exist_ok=True)
    rows = [{"step": i, "seconds": seconds, "supervised_tokens": 100} for i in range(1, n + 1)]
    (root / "train-metrics.jsonl").write_text("".join(json.dumps(r) + "\n" for r in rows) + '{"step": 99, "sec')
    return root


def test_tail_and_guard(tmp_path):
    root = ledger(tmp_path / "arm")
    t = coeval.tail_metrics(root / "train-metrics.jsonl", count=3)
    assert t["step"] == 5 and t["samples"] == 3 and t["median_seconds"] == 2.0 and t["tokens"] == 300
    (tmp_path / "empty.jsonl").write_text("noise\n")
    with pytest.raises(ValueError, match="no completed metrics"):
        coeval.tail_metrics(tmp_path / "empty.jsonl")
    g, roots, snap = coeval.Guard(), {"a": str(root)}, {"a": t}
    now = t["mtime"] + 10
    assert g.reason(roots, snap, 80, 64, now) is None
    assert "GPU headroom" in g.reason(roots, snap, 40, 64, now) and "host headroom" in g.reason(roots, snap, 80, 8, now)
    assert g.reason(roots, snap, 80, 64, now + 1000) == "trainer metrics stale"
    (root / "TRAINING_COMPLETE.json").write_text("{}")
    assert "queue advances" in g.reason(roots, snap, 80, 64, now)


def test_phases_run_in_order_and_yield_when_headroom_falls(tmp_path):
    root = ledger(tmp_path / "arm")
    free = {"gpu": 80.0}
    ev = coeval.CoEvaluator(tmp_path / "out", {"a": str(root)}, free_gpu_gib=lambda: free["gpu"], free_host_gib=lambda: 64.0, poll_seconds=0.05,
                            clock=lambda: (root / "train-metrics.jsonl").stat().st_mtime + 1)
    quick = {"name": "quick", "command": [sys.executable, "-c", "print('scored')"]}
    slow = {"name": "slow", "command": [sys.executable, "-c", "import time; time.sleep(60)"]}
    done = ev.run([quick])
    assert done["complete"] and done["phases"][0]["returncode"] == 0 and done["phases"][0]["trainer_slowdown"] == {"a": 1.0}
    assert b"scored" in (tmp_path / "out" / "phase-0-quick.log").read_bytes()
    with pytest.raises(ValueError, match="already stopped or complete"):
        ev.run([quick])
    ev2 = coeval.CoEvaluator(tmp_path / "out2", {"a": str(root)}, free_gpu_gib=lambda: free["gpu"], free_host_gib=lambda: 64.0, poll_seconds=0.05,
                             clock=lambda: (root / "train-metrics.jsonl").stat().st_mtime + 1)
    free["gpu"] = 10.0
    t0 = time.monotonic()
    stopped = ev2.run([slow, quick])
    assert time.monotonic() - t0 < 20 and not stopped["complete"] and stopped["stopped_at"] == "slow" and "GPU headroom" in stopped["reason"]
    assert stopped["phases"][0]["returncode"] != 0 and len(stopped["phases"]) == 1 and (tmp_path / "out2" / "STOPPED.json").exists()
    failing = {"name": "bad", "command": [sys.executable, "-c", "raise SystemExit(3)"]}
    free["gpu"] = 80.0
    ev3 = coeval.CoEvaluator(tmp_path / "out3", {"a": str(root)}, free_gpu_gib=lambda: 80.0, free_host_gib=lambda: 64.0, poll_seconds=0.05,
                             clock=lambda: (root / "train-metrics.jsonl").stat().st_mtime + 1)
    assert ev3.run([failing, quick])["reason"] == "exit code 3"
