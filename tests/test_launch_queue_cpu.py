"""Launch-request queue: closed schema, git-verified snapshot, once-only processing, single consumer."""
import json
import subprocess
from pathlib import Path

import pytest

from archlab_b200.train import launch_queue as lq


def _schema(root):
    return lq.RequestSchema(launchers=frozenset({"run.sh"}), repo_root=Path(root), requested_from="workbench",
                            allowed_env=frozenset({"NGA_EXPECTED_NODES", "NGA_GPUS_PER_NODE", "NGA_PRECISION", "NGA_OUTPUT_ROOT"}),
                            required_env=frozenset({"NGA_EXPECTED_NODES", "NGA_GPUS_PER_NODE"}),
                            positive_int=frozenset({"NGA_EXPECTED_NODES", "NGA_GPUS_PER_NODE"}),
                            choices={"NGA_PRECISION": {"bf16", "fp4"}}, path_prefix={"NGA_OUTPUT_ROOT": root})


def _repo(tmp_path):
    repo = tmp_path / "snap"
    repo.mkdir()
    (repo / "run.sh").write_text("echo launched $NGA_PRECISION\n")
    for cmd in (["init", "-q"], ["add", "."], ["-c", "user.email=a@b", "-c", "user.name=t", "commit", "-qm", "x"]):
        subprocess.run(["git", "-C", str(repo), *cmd], check=True)
    commit = subprocess.run(["git", "-C", str(repo), "rev-parse", "HEAD"], capture_output=True, text=True).stdout.strip()
    return repo, commit


def _payload(repo, commit, gen="g1", **env):
    return {"schema_version": 1, "generation": gen, "action": "run", "requested_at_utc": "2026-01-01T00:00:00Z",
            "requested_from": "workbench", "repository": {"root": str(repo), "commit": commit}, "launcher": "run.sh",
            "environment": {"NGA_EXPECTED_NODES": "1", "NGA_GPUS_PER_NODE": "8", "NGA_PRECISION": "bf16", **env}}


def test_validation_is_closed(tmp_path):
    repo, commit = _repo(tmp_path)
    s = _schema(tmp_path)
    ok = lq.validate_request(_payload(repo, commit), s)
    assert ok.generation == "g1" and len(ok.digest) == 64
    bad = [dict(_payload(repo, commit), extra=1), _payload(repo, commit, NGA_PRECISION="fp8"), _payload(repo, commit, FOO="1"),
           _payload(repo, "abc"), _payload("/elsewhere", commit), _payload(repo, commit, NGA_GPUS_PER_NODE="0"),
           _payload(repo, commit, NGA_OUTPUT_ROOT="/etc/x"), dict(_payload(repo, commit), requested_at_utc="2026-01-01T00:00:00+08:00")]
    for p in bad:
        with pytest.raises(ValueError):
            lq.validate_request(p, s)
    with pytest.raises(ValueError):
        lq.validate_request(_payload(repo, commit), s, expected_gpus_per_node=4)


def test_controller_runs_once_and_records(tmp_path):
    repo, commit = _repo(tmp_path)
    s, ctl = _schema(tmp_path), tmp_path / "control"
    lq.publish_request(ctl, _payload(repo, commit), s)
    c = lq.Controller(ctl, s, poll_seconds=0.01, expected_nodes=1, expected_gpus_per_node=8)
    assert c.serve(max_polls=2) == 0
    res = json.loads((ctl / "results" / "g1.json").read_text())
    assert res["status"] == "done" and res["returncode"] == 0
    assert "launched bf16" in (ctl / "logs" / "g1.log").read_text()
    events = [json.loads(l)["event"] for l in open(ctl / "events.jsonl")]
    assert events == ["started", "done"]                       # the second poll skipped it
    with pytest.raises(FileExistsError):
        lq.publish_request(ctl, _payload(repo, commit, NGA_PRECISION="fp4"), s)


def test_dirty_snapshot_and_bad_files(tmp_path):
    repo, commit = _repo(tmp_path)
    s, ctl = _schema(tmp_path), tmp_path / "control"
    (repo / "stray.txt").write_text("x")
    lq.publish_request(ctl, _payload(repo, commit, gen="g2"), s)
    (ctl / "requests" / "junk.json").write_text("{not json")
    c = lq.Controller(ctl, s, poll_seconds=0.01)
    c.serve(max_polls=1)
    assert json.loads((ctl / "results" / "g2.json").read_text())["status"] == "failed"
    assert (ctl / "requests" / "junk.rejected").exists()
    c.acquire()
    with pytest.raises(RuntimeError):
        lq.Controller(ctl, s).acquire()
    c.release()
