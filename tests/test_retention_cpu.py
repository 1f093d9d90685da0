"""Checkpoint retention: ordering by cursor, verification before removal, holds, resumable two-phase deletion."""
import json
import os
from pathlib import Path

import pytest
import torch

from archlab_b200.ckpt.formats import write_v41_sharded
from archlab_b200.services import retention as rt


def _save(root: Path, step: int, tokens: int = 0) -> Path:
    state = {"embed.weight": torch.arange(24, dtype=torch.float32).view(6, 4), "norm.weight": torch.ones(4, dtype=torch.bfloat16)}
    path = root / f"step-{step}"
    write_v41_sharded(path, state, cursor={"step": step, "supervised_tokens": tokens}, world_size=2, ep_size=2, expert_fsdp_size=1)
    return path


def _policy(root: Path, **extra) -> rt.Policy:
    return rt.Policy.from_json({"groups": [{"name": "g", "roots": [str(root)]}], **extra})


def test_newest_by_cursor_survives_and_older_complete_saves_go(tmp_path):
    root = (tmp_path / "runs").resolve()
    a, b, c = _save(root, 30), _save(root, 4), _save(root, 100)
    os.utime(c, (1, 1))                                              # modification time must not decide
    unfinished = root / "step-200"
    unfinished.mkdir()
    (unfinished / "rank-00").mkdir()
    dry = rt.Sweeper(tmp_path / "audit").sweep(_policy(root))
    assert dry["errors"] == [] and dry["groups"][0]["newest"] == str(c)
    assert dry["groups"][0]["delete"] == [str(b), str(a)] and a.exists() and b.exists()
    done = rt.Sweeper(tmp_path / "audit", apply=True).sweep(_policy(root))
    assert not a.exists() and not b.exists() and c.exists() and unfinished.exists()
    receipts = done["groups"][0]["removed"]
    assert all(r["complete"] and r["bytes"] > 0 for r in receipts)
    assert json.loads((root / "LATEST.json").read_text())["path"] == str(c)
    archived = list((tmp_path / "audit" / "deleted").glob("*/rank-00/MANIFEST.json"))
    assert len(archived) == 2                                         # what was removed stays on record
    assert list((tmp_path / "audit").glob("verified-*.json"))


def test_holds_keep_a_save(tmp_path):
    root = (tmp_path / "runs").resolve()
    saves = {s: _save(root, s) for s in (1, 2, 3, 4, 5, 9)}
    (saves[1] / "PINNED.json").write_text("{}")
    (saves[2] / "EVAL_PENDING.json").write_text("{}")
    (saves[3] / ".checkpoint-readers").mkdir()
    (saves[3] / ".checkpoint-readers" / "eval-7.json").write_text("{}")
    policy = _policy(root, protected={str(saves[4]): "paper figure"}, protected_steps=[5])
    out = rt.Sweeper(tmp_path / "audit", apply=True).sweep(policy)
    assert out["groups"][0]["delete"] == [] and all(p.exists() for p in saves.values())
    assert sorted(out["groups"][0]["held"].values()) == sorted(["PINNED.json", "EVAL_PENDING.json", "reader lease", "protected path", "protected step"])


def test_a_damaged_survivor_blocks_removal(tmp_path):
    root = (tmp_path / "runs").resolve()
    old, new = _save(root, 1), _save(root, 2)
    victim = next((new / "rank-01").glob("t00000-c000.pt"))
    victim.write_bytes(b"short")
    out = rt.Sweeper(tmp_path / "audit", apply=True).sweep(_policy(root))
    assert out["groups"] == [] and "bad payload length" in out["errors"][0]["error"] and old.exists()


def test_interrupted_removal_is_finished_and_symlinks_are_refused(tmp_path):
    root = (tmp_path / "runs").resolve()
    old, new = _save(root, 1), _save(root, 2)
    audit = tmp_path / "audit"
    key = rt._key(old)
    staged = old.with_name(rt.STAGED_PREFIX + key)
    (audit / "deleted" / key).mkdir(parents=True)
    (audit / "deleted" / key / "RECEIPT.json").write_text(json.dumps(
        {"original": str(old), "staged": str(staged), "replacement": str(new), "bytes": 1, "started_utc": "t", "complete": False}))
    old.rename(staged)                                               # the sweeper died right after the rename
    out = rt.Sweeper(audit, apply=True).sweep(_policy(root))
    assert out["resumed"] == [str(staged)] and not staged.exists() and new.exists()
    assert json.loads((audit / "deleted" / key / "RECEIPT.json").read_text())["complete"] is True
    older = _save(root, 0)
    (older / "rank-00" / "escape").symlink_to(tmp_path)
    out = rt.Sweeper(audit, apply=True).sweep(_policy(root))
    assert "symlink inside deletion candidate" in out["errors"][0]["error"] and older.exists()


def test_cli_dry_run_and_lock(tmp_path, capsys):
    root = (tmp_path / "runs").resolve()
    _save(root, 1), _save(root, 2)
    cfg = tmp_path / "policy.json"
    cfg.write_text(json.dumps({"groups": [{"name": "g", "roots": [str(root)]}]}))
    assert rt.main(["--config", str(cfg), "--audit", str(tmp_path / "audit")]) == 0
    assert json.loads(capsys.readouterr().out)["groups"][0]["delete"] == [str(root / "step-1")]
    with pytest.raises(SystemExit):
        rt.main(["--config", str(cfg), "--audit", str(tmp_path / "audit"), "--interval", "0.1"])


def test_checkpoint_receipt_samples_content(tmp_path):
    import pytest
    import torch

    from archlab_b200.ckpt.formats import write_v41_sharded
    from archlab_b200.services.retention import checkpoint_receipt

    state = {"embed.weight": torch.arange(12, dtype=torch.float32).view(6, 2), "mid.weight": torch.ones(4, 2), "head.weight": torch.full((6, 2), 3.0)}
    write_v41_sharded(tmp_path / "ck", state, cursor={"step": 5, "supervised_tokens": 50}, world_size=2, ep_size=2, expert_fsdp_size=1)
    receipt = checkpoint_receipt(tmp_path / "ck", sample_ranks=(0, 1))
    assert receipt["passed"] and [s["name"] for s in receipt["representative_checksums"]] == ["embed.weight", "head.weight"] * 2
    manifest = tmp_path / "ck" / "rank-01" / "MANIFEST.json"
    import json
    body = json.loads(manifest.read_text())
    chunk = next(t for t in body["tensors"] if t["name"] == "head.weight")["chunks"][0]
    torch.save(torch.zeros(chunk["elements"]), manifest.parent / chunk["file"])                  # same length, other content
    with pytest.raises(ValueError, match="payload checksum mismatch: rank 1 head.weight"):
        checkpoint_receipt(tmp_path / "ck", sample_ranks=(0, 1))
    assert checkpoint_receipt(tmp_path / "ck", sample_tensors=("mid.weight",))["representative_checksums"][0]["name"] == "mid.weight"
    with pytest.raises(ValueError, match="not in the checkpoint"):
        checkpoint_receipt(tmp_path / "ck", sample_tensors=("absent",))
