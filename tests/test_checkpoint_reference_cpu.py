"""Checkpoint references: metadata-only bundles, deterministic archives, one attachment per checkpoint, availability catalogue."""
import json
import shutil
import zipfile

import pytest
import torch

from archlab_b200.ckpt.formats import write_v41_sharded
from archlab_b200.services import checkpoint_reference as cr


def _checkpoint(path, step, variant="normal"):
    write_v41_sharded(path, {"w": torch.arange(16, dtype=torch.float32).view(8, 2)}, cursor={"step": step, "supervised_tokens": step * 100},
                      world_size=2, ep_size=2, expert_fsdp_size=1, variant=variant)
    return path


def test_bundle_holds_metadata_only_and_is_deterministic(tmp_path):
    ck = _checkpoint(tmp_path / "run" / "checkpoints" / "step-10", 10)
    ref = cr.make_bundle(ck, tmp_path / "b1", "normal")
    cr.make_bundle(ck, tmp_path / "b2", "normal")
    assert (tmp_path / "b1" / "rank-manifests.zip").read_bytes() == (tmp_path / "b2" / "rank-manifests.zip").read_bytes()
    assert sorted(p.name for p in (tmp_path / "b1").iterdir()) == ["COMPLETE.json", "METADATA_SHA256.json", "REFERENCE.json", "RESTORE.md", "rank-manifests.zip"]
    assert ref["weights_uploaded"] is False and ref["rank_manifests"] == 2 and ref["tensor_payload_chunks_referenced"] == 2 and ref["cursor"]["step"] == 10
    with zipfile.ZipFile(tmp_path / "b1" / "rank-manifests.zip") as z:
        assert z.namelist() == ["rank-00/MANIFEST.json", "rank-01/MANIFEST.json"]
    assert cr.verify_bundle(tmp_path / "b1")["source_path"] == str(ck.resolve())
    assert "step: **10**" in (tmp_path / "b1" / "RESTORE.md").read_text()
    (tmp_path / "b1" / "COMPLETE.json").write_text("{}")
    with pytest.raises(ValueError, match="marker changed"):
        cr.verify_bundle(tmp_path / "b1")


def test_inconsistent_checkpoints_are_refused(tmp_path):
    ck = _checkpoint(tmp_path / "c", 10)
    with pytest.raises(ValueError, match="wrong checkpoint format or variant"):
        cr.make_bundle(ck, tmp_path / "b", "simplicial")
    m = json.loads((ck / "rank-01" / "MANIFEST.json").read_text())
    (ck / "rank-01" / "MANIFEST.json").write_text(json.dumps({**m, "cursor": {"step": 9, "supervised_tokens": 900}}))
    with pytest.raises(ValueError, match="identity mismatch"):
        cr.make_bundle(ck, tmp_path / "b", "normal")
    marker = json.loads((ck / "COMPLETE.json").read_text())
    (ck / "COMPLETE.json").write_text(json.dumps({**marker, "manifests": ["rank-00/MANIFEST.json", "../outside.json"]}))
    with pytest.raises(ValueError, match="unsafe manifest path"):
        cr.make_bundle(ck, tmp_path / "b", "normal")


def test_sidecar_attaches_each_complete_checkpoint_once(tmp_path):
    root = tmp_path / "run"
    _checkpoint(root / "checkpoints" / "step-20", 20)
    _checkpoint(root / "checkpoints" / "step-5", 5)
    (root / "checkpoints" / "step-30").mkdir()                                   # still being written: no marker
    _checkpoint(root / "checkpoints" / "step-40", 40, variant="simplicial")     # another arm's checkpoint in the wrong place
    sink = cr.log_artifacts_to_directory(tmp_path / "store")
    side = cr.CheckpointAttachments(sink, tmp_path / "state.json")
    spec = {"run_id": "0001-run", "root": str(root), "variant": "normal"}
    first = side.sync(spec)
    assert first["attached"] == ["step-5", "step-20"] and first["skipped"][0]["checkpoint"] == "step-40"
    assert (tmp_path / "store" / "0001-run" / "artifacts" / "checkpoints" / "step-20" / "REFERENCE.json").exists()
    assert cr.CheckpointAttachments(sink, tmp_path / "state.json").sync(spec)["attached"] == []          # state survives a restart
    shutil.rmtree(root / "checkpoints" / "step-5")                               # pruned by retention later
    _checkpoint(root / "checkpoints" / "step-50", 50)
    assert side.sync(spec)["attached"] == ["step-50"]
    catalog = json.loads((root / "checkpoints" / "CATALOG.json").read_text())["checkpoints"]
    assert catalog["step-5"]["source_available"] is False and catalog["step-50"]["source_available"] is True
