import json
import subprocess

import pytest
import torch

from archlab_b200.contracts import provenance as pv, registry as rg, source_compat as sc


def test_dataset_manifest_roundtrip_and_tamper(tmp_path):
    root = tmp_path / "data"
    (root / "sub").mkdir(parents=True)
    (root / "a.bin").write_bytes(b"abc")
    (root / "sub" / "b.bin").write_bytes(b"defg")
    m = pv.create_dataset_manifest(root, dataset="toy", revision="r1")
    path = tmp_path / "manifest.json"
    pv.write_dataset_manifest(path, m)
    out = pv.verify_dataset_manifest(root, path, mode="full")
    assert out["files"] == 2 and out["bytes"] == 7 and out["identity_sha256"] == m.identity_sha256
    (root / "a.bin").write_bytes(b"abd")                        # same size, other content
    pv.verify_dataset_manifest(root, path, mode="metadata")
    with pytest.raises(pv.ProvenanceError):
        pv.verify_dataset_manifest(root, path, mode="full")
    (root / "extra.bin").write_bytes(b"x")
    with pytest.raises(pv.ProvenanceError):
        pv.verify_dataset_manifest(root, path)
    pv.verify_dataset_manifest(root, path, required_files=["sub/b.bin"])
    with pytest.raises(pv.ProvenanceError):
        pv.DatasetFile("../evil", 1, "0" * 64).validate()


def test_legacy_ledger_loads(tmp_path):
    (tmp_path / "x").write_bytes(b"1")
    digest = pv.sha256_file(tmp_path / "x")
    ledger = tmp_path / "SHA256SUMS"
    ledger.write_text(f"{digest}  ./x\n")
    m = pv.load_dataset_manifest(ledger, dataset_root_name="d")
    assert m.files[0].path == "x" and m.files[0].size is None


def test_source_provenance_sees_dirty_tree(tmp_path):
    run = lambda *a: subprocess.run(["git", *a], cwd=tmp_path, check=True, capture_output=True)
    run("init", "-q")
    run("config", "user.email", "a@b")
    run("config", "user.name", "n")
    (tmp_path / "f.py").write_text("x = 1\n")
    run("add", ".")
    run("commit", "-qm", "c")
    clean = pv.source_provenance(tmp_path)
    assert not clean["source_dirty"] and len(clean["source_commit"]) == 40
    (tmp_path / "g.py").write_text("y = 2\n")
    dirty = pv.source_provenance(tmp_path)
    assert dirty["source_dirty"] and dirty["source_untracked_files"] == ["g.py"]
    assert dirty["source_worktree_sha256"] != clean["source_worktree_sha256"]


def test_tensor_hash_depends_on_bits_names_and_dtype():
    a = {"w": torch.arange(6.0).view(2, 3), "b": torch.zeros(2, dtype=torch.bfloat16)}
    h = pv.hash_named_tensors(a.items())
    assert h == pv.hash_named_tensors(reversed(list(a.items())))
    assert h != pv.hash_named_tensors({"w": a["w"].clone().add_(1), "b": a["b"]}.items())
    assert h != pv.hash_named_tensors({"w": a["w"], "b": a["b"].float()}.items())
    assert pv.hash_named_tensors(a.items(), include_names={"w"}) != h
    with pytest.raises(pv.ProvenanceError):
        pv.hash_named_tensors(a.items(), include_names={"missing"})


def test_campaign_grid_is_complete_and_commands_are_exact(tmp_path):
    path = tmp_path / "campaign.json"
    rg.write_manifest(path)
    assert rg.verify_manifest(path) == {"runs": 3 * 16 * 3, "sizes": 3, "variants": 16, "seeds": 3}
    runs = rg.load_runs(path)
    run = rg.find_run(runs, "100m", "kda", 1)
    cmd = run.command(run_name="r")
    assert cmd[:3] == ["python", "-m", "archlab_b200.train.base_train"] and "--seed=1" in cmd and "--kda-pattern=KKKG" in cmd and "--arch-family=kimi_kda" in cmd
    data = json.loads(path.read_text())
    data["runs"].pop()
    path.write_text(json.dumps(data))
    with pytest.raises(ValueError):
        rg.verify_manifest(path)


def test_capabilities_fail_closed():
    rg.require_backend_support("baseline", "megatron")
    rg.require_backend_support("xielu", "speedrun")
    with pytest.raises(ValueError):
        rg.require_backend_support("xielu", "megatron")
    with pytest.raises(ValueError):
        rg.require_backend_support("nope", "speedrun")
    assert len(rg.capability_rows()) == len(rg.CAPABILITIES)


def test_formatting_only_change_detection(tmp_path):
    before = "def f(a,b):\n    return a+b\n"
    assert sc.formatting_only_change(before, "def f(a, b):\n    return a + b\n")
    assert not sc.formatting_only_change(before, "def f(a, b):\n    return a - b\n")
    (tmp_path / "m.py").write_text(before)
    sealed = {"m.py": sc.ast_sha256(before)}
    sc.prove_compatible(sealed, tmp_path)
    (tmp_path / "m.py").write_text("def f(a, b):\n    return a * b\n")
    with pytest.raises(ValueError):
        sc.prove_compatible(sealed, tmp_path)
