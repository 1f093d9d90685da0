"""Run-level tracking sync: exactly-once delivery, resumable batches, source-change refusal."""
import json
from pathlib import Path

import pytest

from archlab_b200.services import tracking as tk


def _run(tmp_path: Path, steps: int, commit: str = "c1", start: int = 1) -> dict:
    root = tmp_path / "run"
    root.mkdir(exist_ok=True)
    (root / "RUN_CONTRACT.json").write_text(json.dumps({"project_commit": commit, "world_size": 8, "optimizer": "muon_split"}))
    with (root / "train-metrics.jsonl").open("a") as f:
        for s in range(start, start + steps):
            f.write(json.dumps({"step": s, "loss": 5.0 - 0.01 * s, "supervised_tokens": 100, "consumed_supervised_tokens": 100 * s,
                                "seconds": 0.5, "learning_rate": 1e-3, "gradient_norm_before_clip": 1.5, "max_memory_allocated_gib": 40.0}) + "\n")
    return {"id": "src-1", "name": "d20", "path": str(root), "phase": "pretrain", "variant": "normal"}


def _points(store, run_id, metric):
    return [p for p in map(json.loads, (store.root / run_id / "points.jsonl").read_text().splitlines()) if p[0] == metric]


def test_exactly_once_across_passes_and_restarts(tmp_path):
    spec = _run(tmp_path, 3)
    store = tk.FileTrackingStore(tmp_path / "store")
    sync = tk.TrackingSync(store, tmp_path / "state.json")
    first = sync.sync_run(spec)
    assert first["new_updates"] == 3 and first["last_step"] == 3
    assert sync.sync_run(spec)["new_updates"] == 0
    _run(tmp_path, 2, start=4)
    with (Path(spec["path"]) / "train-metrics.jsonl").open("a") as f:
        f.write('{"step": 6, "loss"')                                  # a writer is mid-line
    again = tk.TrackingSync(store, tmp_path / "state.json").sync_run(spec)      # a new process picks up the cursor
    assert again["new_updates"] == 2
    run_id = store.find_runs("src-1")[0]
    assert [p[2] for p in _points(store, run_id, "train/cross_entropy")] == [1, 2, 3, 4, 5]
    assert _points(store, run_id, "train/cross_entropy_by_tokens")[-1][2] == 500
    assert _points(store, run_id, "perf/target_tokens_per_second")[0][1] == 200.0
    meta = json.loads((store.root / run_id / "meta.json").read_text())
    assert meta["params"]["gpu_type"] == "NVIDIA B200" and meta["tags"]["archlab_source_id"] == "src-1"


def test_a_crash_between_write_and_cursor_resends_identical_points(tmp_path):
    spec = _run(tmp_path, 130)                                          # three batches: a back-fill
    store = tk.FileTrackingStore(tmp_path / "store")

    class Dies(tk.FileTrackingStore):
        calls = 0

        def log_points(self, run_id, points):
            super().log_points(run_id, points)
            Dies.calls += 1
            if Dies.calls == 2:
                raise OSError("connection lost after the server stored the batch")

    with pytest.raises(OSError):
        tk.TrackingSync(Dies(tmp_path / "store"), tmp_path / "state.json").sync_run(spec)
    state = json.loads((tmp_path / "state.json").read_text())["runs"]["src-1"]
    assert state["last_step"] == 60 and state["pending_batch"]["first_step"] == 61
    out = tk.TrackingSync(store, tmp_path / "state.json").sync_run(spec)
    assert out["new_updates"] == 70
    run_id = store.find_runs("src-1")[0]
    ce = _points(store, run_id, "train/cross_entropy")
    assert [p[2] for p in ce] == list(range(1, 131)) and len({p[3] for p in ce}) == 1      # one back-fill timestamp, no duplicates


def test_refusals(tmp_path):
    spec = _run(tmp_path, 3)
    store = tk.FileTrackingStore(tmp_path / "store")
    sync = tk.TrackingSync(store, tmp_path / "state.json")
    sync.sync_run(spec)
    (Path(spec["path"]) / "RUN_CONTRACT.json").write_text(json.dumps({"project_commit": "c2"}))
    with pytest.raises(ValueError, match="qualified continuation"):
        sync.sync_run(spec)
    (Path(spec["path"]) / "SOURCE_TRANSITION.json").write_text(json.dumps(
        {"from_commit": "c1", "to_commit": "c2", "training_math_unchanged": True, "cursor": {"step": 3}}))
    assert sync.sync_run(spec)["new_updates"] == 0
    assert json.loads((store.root / store.find_runs("src-1")[0] / "meta.json").read_text())["tags"]["archlab.current_source_commit"] == "c2"
    ledger = Path(spec["path"]) / "train-metrics.jsonl"
    lines = ledger.read_text().splitlines()
    ledger.write_text("\n".join(lines[:2]) + "\n")
    with pytest.raises(ValueError, match="ahead of source"):
        sync.sync_run(spec)
    ledger.write_text("\n".join([lines[0], lines[2]]) + "\n")
    with pytest.raises(ValueError, match="not contiguous"):
        sync.sync_run(spec)
    store.create_run("src-2", "a", {}), store.create_run("src-2", "b", {})
    out = sync.sync_all([{**spec, "id": "src-2"}, {"id": "queued", "name": "q", "path": str(tmp_path / "none"), "defer_until_training": True}])
    assert out["runs"] == [{"id": "queued", "state": "queued", "new_updates": 0}] and "src-2" in json.dumps(out["errors"])


def test_validation_rows_follow_the_token_cursor_once(tmp_path):
    spec = _run(tmp_path, 4)
    (Path(spec["path"]) / "validation.jsonl").write_text('{"step": 0, "loss": 9.0}\n{"step": 4, "loss": 4.5}\n')
    store = tk.FileTrackingStore(tmp_path / "store")
    sync = tk.TrackingSync(store, tmp_path / "state.json")
    assert sync.sync_run(spec)["validation_points"] == 4 and sync.sync_run(spec)["validation_points"] == 0
    by_tokens = _points(store, store.find_runs("src-1")[0], "eval/cross_entropy_by_tokens")
    assert [(p[1], p[2]) for p in by_tokens] == [(9.0, 0), (4.5, 400)]
    reg = tmp_path / "registry.json"
    reg.write_text(json.dumps([spec]))
    assert tk.main(["--registry", str(reg), "--store", str(tmp_path / "store"), "--state", str(tmp_path / "state.json")]) == 0
