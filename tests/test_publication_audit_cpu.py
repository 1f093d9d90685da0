"""Publication audit over a committed tree: rule table, secrets by name only, manifest."""
import hashlib
import json
import os
import subprocess

import pytest

from archlab_b200.services import publication_audit as pa


def _git(root, *args):
    env = {**os.environ, "GIT_AUTHOR_NAME": "t", "GIT_AUTHOR_EMAIL": "t@t", "GIT_COMMITTER_NAME": "t", "GIT_COMMITTER_EMAIL": "t@t"}
    subprocess.run(["git", "-C", str(root), *args], check=True, capture_output=True, env=env)


@pytest.fixture
def repo(tmp_path):
    _git(tmp_path, "init", "-q")
    (tmp_path / "archlab_b200").mkdir()
    (tmp_path / "archlab_b200" / "a.py").write_text("x = 1\n")
    (tmp_path / "README.md").write_text("hello\n")
    (tmp_path / ".gitignore").write_text("_scratch/\n")
    _git(tmp_path, "add", "-A")
    _git(tmp_path, "commit", "-qm", "base")
    return tmp_path


def test_clean_tree_passes_with_a_manifest(repo, tmp_path, capsys):
    out = pa.audit_tree(repo)
    assert out["passed"] and out["files"] == 3 and out["findings"] == []
    row = next(m for m in out["manifest"] if m["path"] == "README.md")
    assert row == {"path": "README.md", "bytes": 6, "sha256": hashlib.sha256(b"hello\n").hexdigest()}
    assert pa.main(["--root", str(repo), "--output", str(tmp_path / "audit.json")]) == 0
    assert json.loads((tmp_path / "audit.json").read_text())["revision"] == out["revision"]


def test_findings_name_rules_and_never_the_secret(repo, tmp_path):
    (repo / "archlab_b200" / "weights.safetensors").write_bytes(b"\0" * 10)
    (repo / "runs").mkdir()
    (repo / "runs" / "notes.md").write_text("n\n")
    (repo / "scratchpad").mkdir()
    (repo / "scratchpad" / "x.py").write_text("y = 2\n")
    token = "ghp_" + "A" * 40
    (repo / "tests").mkdir()
    (repo / "tests" / "conf.py").write_text(f"TOKEN = '{token}'\nURL = 'https://user:hunter2@host/x'\n")
    os.symlink("a.py", repo / "archlab_b200" / "link.py")
    (repo / "archlab_b200" / "big.txt").write_bytes(b"a" * (5 * 1024 * 1024 + 1))
    (repo / ".env.local").write_text("K=V\n")
    _git(repo, "add", "-A")
    _git(repo, "commit", "-qm", "bad")
    out = pa.audit_tree(repo)
    found = {f["path"]: f["reasons"] for f in out["findings"]}
    assert found["archlab_b200/weights.safetensors"] == ["data_or_secret_file"]
    assert found["runs/notes.md"] == ["unapproved_root", "workspace_artifact"]
    assert found["scratchpad/x.py"] == ["unapproved_root"]
    assert found["tests/conf.py"] == ["github_token", "credential_url"]
    assert found["archlab_b200/link.py"] == ["non_regular_file"]
    assert found["archlab_b200/big.txt"] == ["oversize_blob"]
    assert found[".env.local"] == ["unapproved_root", "data_or_secret_file"]
    assert not out["passed"] and token not in json.dumps(out) and "hunter2" not in json.dumps(out)
    assert pa.main(["--root", str(repo), "--output", str(tmp_path / "a.json")]) == 1
    # the previous revision is still clean: the audit reads the named tree, not the work tree
    assert pa.audit_tree(repo, "HEAD~1")["passed"]
