"""Bulk offload planning and two-phase directory migration (copy-verify, then swap for a link with a restorable backup)."""
import json

import pytest

from archlab_b200.services import migration as mg


def _tree(root):
    (root / "model" / "sub").mkdir(parents=True)
    (root / "model" / "a.safetensors").write_bytes(b"a" * 100)
    (root / "model" / "sub" / "b.bin").write_bytes(b"b" * 50)
    (root / "model" / "config.json").write_text("{}")
    return root / "model"


def test_plan_selects_finished_payloads_only(tmp_path):
    src = tmp_path / "results"
    (src / "run" / "checkpoints" / "step-10").mkdir(parents=True)
    (src / "run" / "checkpoints" / "step-10" / "w.pt").write_bytes(b"x" * 64)
    (src / "run" / "checkpoints" / "step-10" / "COMPLETE.json").write_text("{}")
    (src / "run" / "checkpoints" / "step-20").mkdir()
    (src / "run" / "checkpoints" / "step-20" / "w.pt").write_bytes(b"x" * 64)              # no completion marker
    (src / "run" / "metrics.jsonl").write_text("{}\n" * 40)
    (src / "run" / "small.npy").write_bytes(b"x" * 4)
    (src / "repo" / ".git").mkdir(parents=True)
    (src / "repo" / "big.bin").write_bytes(b"x" * 64)
    (src / "busy").mkdir()
    (src / "busy" / mg.IN_USE_MARKER).write_text("{}")
    (src / "busy" / "w.pt").write_bytes(b"x" * 64)
    (src / "run" / ".retention-delete-1").mkdir()
    (src / "run" / ".retention-delete-1" / "w.pt").write_bytes(b"x" * 64)
    (src / "run" / "link.pt").symlink_to(src / "run" / "checkpoints" / "step-10" / "w.pt")
    tasks, summary = mg.offload_plan(src, tmp_path / "bulk", minimum_bytes=16)
    assert [t["source"] for t in tasks] == [str(src / "run" / "checkpoints" / "step-10" / "w.pt")]
    assert tasks[0]["destination"] == str(tmp_path / "bulk" / "run" / "checkpoints" / "step-10" / "w.pt")
    assert summary["files"] == 1 and summary["repositories_skipped"] == 1 and len(summary["incomplete_checkpoints_skipped"]) == 1
    assert summary["active_reader_trees_skipped"] == [str(src / "busy")]


def test_two_phase_migration_and_restore_on_failure(tmp_path):
    model = _tree(tmp_path / "nas")
    bulk = tmp_path / "bulk" / "model"
    bulk.mkdir(parents=True)
    (bulk / "unrelated.txt").write_text("keep")
    (bulk / "sub").mkdir()
    (bulk / "sub" / "b.bin").write_bytes(b"b" * 50)                       # identical file already there: reused
    m = mg.TreeMigration(tmp_path / "journal.json")
    with pytest.raises(ValueError, match="only a fully verified"):
        m._save({"phase": "copying"}) or m.commit()
    state = m.prepare(model, bulk)
    assert state["phase"] == "verified" and state["files"]["sub/b.bin"]["reused_existing"] and not state["files"]["a.safetensors"]["reused_existing"]

    def boom():
        raise OSError("link publication failed")
    with pytest.raises(OSError):
        m.commit(after_backup=boom)
    assert model.is_dir() and not model.is_symlink() and (model / "a.safetensors").read_bytes() == b"a" * 100
    assert m.state()["phase"] == "verified" and not list(model.parent.glob(".model.*"))
    done = m.commit()
    assert done["phase"] == "complete" and model.is_symlink() and model.resolve() == bulk.resolve()
    assert (model / "sub" / "b.bin").read_bytes() == b"b" * 50 and (bulk / "unrelated.txt").read_text() == "keep"
    assert not list(model.parent.glob(".model.backup-*"))


def test_refusals(tmp_path):
    model = _tree(tmp_path / "nas")
    bulk = tmp_path / "bulk"
    bulk.mkdir()
    m = mg.TreeMigration(tmp_path / "j.json")
    with pytest.raises(ValueError, match="disjoint"):
        m.prepare(model, model / "sub")
    with pytest.raises(ValueError, match="real directory"):
        m.prepare(model, tmp_path / "missing")
    (bulk / "a.safetensors").write_bytes(b"z" * 100)
    with pytest.raises(ValueError, match="collision"):
        m.prepare(model, bulk)
    (bulk / "a.safetensors").unlink()
    (model / "odd").symlink_to(model / "config.json")
    with pytest.raises(ValueError, match="unsupported source entry"):
        m.prepare(model, bulk)
    (model / "odd").unlink()
    (tmp_path / "nas" / mg.IN_USE_MARKER).write_text("{}")
    with pytest.raises(ValueError, match="active readers"):
        m.prepare(model, bulk)
    (tmp_path / "nas" / mg.IN_USE_MARKER).unlink()
    m.prepare(model, bulk)
    (model / "config.json").write_text('{"changed": 1}')
    with pytest.raises(ValueError, match="source changed after verification"):
        m.commit()


def test_watcher_picks_up_new_finished_payloads(tmp_path):
    src, dst = tmp_path / "results", tmp_path / "bulk"
    step = src / "run" / "checkpoints" / "step-10"
    step.mkdir(parents=True)
    (step / "w.pt").write_bytes(b"a" * 64)
    (step / "COMPLETE.json").write_text("{}")
    pending = src / "run" / "checkpoints" / "step-20"
    pending.mkdir()
    (pending / "w.pt").write_bytes(b"b" * 64)
    kw = dict(cycles=1, minimum_bytes=16, sleep=lambda s: None)
    first = mg.offload_watch(src, dst, tmp_path / "plan.jsonl", tmp_path / "journal.db", **kw)
    assert first["state"] == "caught_up" and first["new_files"] == 1 and first["transferred"] == 1
    assert (dst / "run" / "checkpoints" / "step-10" / "w.pt").read_bytes() == b"a" * 64 and not (dst / "run" / "checkpoints" / "step-20").exists()
    (pending / "COMPLETE.json").write_text("{}")                                 # the second checkpoint finishes
    second = mg.offload_watch(src, dst, tmp_path / "plan.jsonl", tmp_path / "journal.db", **kw)
    assert second["new_files"] == 1 and second["transferred"] == 1 and (dst / "run" / "checkpoints" / "step-20" / "w.pt").exists()
    third = mg.offload_watch(src, dst, tmp_path / "plan.jsonl", tmp_path / "journal.db", **kw)
    assert third["new_files"] == 0 and third["transferred"] == 0
    assert json.loads((tmp_path / "OFFLOAD_WATCH_STATUS.json").read_text())["state"] == "caught_up"
    assert mg.grow_plan(tmp_path / "plan.jsonl", [{"source": str(step / "w.pt"), "destination": "x", "bytes": 1}]) == 0
