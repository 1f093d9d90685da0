"""Attaching checkpoints to tracked runs BY REFERENCE: a small metadata bundle travels to the tracking store, the weight,
optimizer and RNG payloads stay where they are and are never opened, copied or modified.

``make_bundle(checkpoint, destination, variant)`` reads a sharded checkpoint's completion marker and every rank manifest
(paths confined to the checkpoint, no symlinks), checks that ranks, contract and cursor agree, re-reads the marker at
the end (a checkpoint pruned or replaced meanwhile is refused), and writes

    COMPLETE.json          the marker, byte for byte
    rank-manifests.zip     all rank manifests, fixed timestamps and order (the same checkpoint gives the same bytes)
    REFERENCE.json         where the payloads live, which mesh restores them, what was and was not uploaded
    METADATA_SHA256.json   digests of the marker and of every manifest
    RESTORE.md             instructions for a person

``CheckpointAttachments`` is the sidecar: for each run specification it finds complete checkpoints not yet attached,
bundles them in a scratch directory, hands the bundle to the tracking store, records the attachment in its state file
(one writer at a time) and keeps ``CATALOG.json`` with the last observed availability of every referenced source.
(Reference: src/archlab/tracking/mlflow_checkpoints.py:31-290.)
"""
from __future__ import annotations

import hashlib
import json
import shutil
import tempfile
import time
import zipfile
from pathlib import Path

from ..contracts.substrate import atomic_write_json
from .tracking import SingleWriterLock

REFERENCE_FORMAT = "archlab-checkpoint-reference-v1"


def _sha(data: bytes) -> str:
    return hashlib.sha256(data).hexdigest()


def confined_file(root: Path, relative: str) -> Path:
    name = Path(relative)
    if name.is_absolute() or ".." in name.parts:
        raise ValueError("unsafe manifest path")
    path = root / name
    if path.is_symlink() or not path.resolve().is_relative_to(root.resolve()):
        raise ValueError("a manifest escapes its checkpoint")
    return path


def make_bundle(checkpoint, destination, expected_variant: str, *, checkpoint_format: str = "archlab-v41-full-sharded-v1",
                storage: dict | None = None) -> dict:
    checkpoint, destination = Path(checkpoint).resolve(), Path(destination)
    raw = (checkpoint / "COMPLETE.json").read_bytes()
    marker = json.loads(raw)
    if marker["format"] != checkpoint_format or marker["contract"]["variant"] != expected_variant:
        raise ValueError("wrong checkpoint format or variant")
    world = marker["world_size"]
    names = marker.get("manifests") or [f"rank-{r:02d}/MANIFEST.json" for r in range(world)]
    if len(names) != world or len(set(names)) != world:
        raise ValueError("incomplete rank manifest set")
    manifests, digests, chunks, optimizer_files = {}, {"COMPLETE.json": _sha(raw)}, 0, 0
    for rank, relative in enumerate(names):
        data = confined_file(checkpoint, relative).read_bytes()
        m = json.loads(data)
        if m["rank"] != rank or any(m[k] != marker[k] for k in ("world_size", "cursor", "contract")):
            raise ValueError("rank manifest identity mismatch")
        manifests[relative], digests[relative] = data, _sha(data)
        chunks += sum(len(t["chunks"]) for t in m["tensors"])
        optimizer_files += len(m.get("optimizer_states", []))
    if (checkpoint / "COMPLETE.json").read_bytes() != raw:
        raise ValueError("the checkpoint changed while its metadata was read")
    destination.mkdir(parents=True, exist_ok=True)
    (destination / "COMPLETE.json").write_bytes(raw)
    with zipfile.ZipFile(destination / "rank-manifests.zip", "w", compression=zipfile.ZIP_DEFLATED, compresslevel=6) as archive:
        for relative, data in manifests.items():
            info = zipfile.ZipInfo(relative, date_time=(1980, 1, 1, 0, 0, 0))
            info.compress_type = zipfile.ZIP_DEFLATED
            archive.writestr(info, data)
    contract = marker["contract"]
    reference = {"format": REFERENCE_FORMAT, "attachment_mode": "reference-and-manifests", "weights_uploaded": False,
                 "optimizer_payloads_uploaded": False, "rng_payloads_uploaded": False, "source_path": str(checkpoint),
                 "source_uri": checkpoint.as_uri(), "storage": storage or {"resolved_path": str(checkpoint)},
                 "checkpoint_format": marker["format"], "variant": expected_variant, "cursor": marker["cursor"], "world_size": world,
                 "expert_parallel": contract.get("ep_size"), "source_commit": contract.get("project_commit"),
                 "checkpoint_marker_sha256": _sha(raw), "rank_manifests": world, "tensor_payload_chunks_referenced": chunks,
                 "optimizer_payload_files_referenced": optimizer_files,
                 "rank_manifests_zip_sha256": _sha((destination / "rank-manifests.zip").read_bytes()),
                 "metadata_validation": "rank identities, contracts and cursors checked; payloads not re-read",
                 "restore_requires": "the original payload files on the source mount and the trained mesh"}
    atomic_write_json(destination / "REFERENCE.json", reference)
    atomic_write_json(destination / "METADATA_SHA256.json", digests)
    cursor = marker["cursor"]
    (destination / "RESTORE.md").write_text(
        f"# Checkpoint reference: {checkpoint.name}\n\n**Metadata only.** Weight, optimizer and RNG payloads remain at `{checkpoint}`.\n\n"
        f"- variant: **{expected_variant}**\n- optimizer step: **{cursor.get('step', 0):,}**\n"
        f"- supervised tokens: **{cursor.get('supervised_tokens', 0):,}**\n- restore mesh: **{world} ranks**\n"
        f"- source commit: `{contract.get('project_commit')}`\n\n"
        "`COMPLETE.json` holds the run contract and the data cursor; `rank-manifests.zip` holds every rank manifest with the "
        "SHA-256 of each weight chunk; `METADATA_SHA256.json` verifies both.  The bundle alone cannot restore the model: "
        "resume with `--resume <source path>` on a machine that sees the source mount.  Variants are not interchangeable.\n")
    return reference


def verify_bundle(bundle) -> dict:
    bundle = Path(bundle)
    digests = json.loads((bundle / "METADATA_SHA256.json").read_text())
    reference = json.loads((bundle / "REFERENCE.json").read_text())
    marker_sha = _sha((bundle / "COMPLETE.json").read_bytes())
    if marker_sha != digests["COMPLETE.json"] or marker_sha != reference["checkpoint_marker_sha256"]:
        raise ValueError("the bundled marker changed")
    if _sha((bundle / "rank-manifests.zip").read_bytes()) != reference["rank_manifests_zip_sha256"]:
        raise ValueError("the bundled manifests changed")
    with zipfile.ZipFile(bundle / "rank-manifests.zip") as archive:
        for name in archive.namelist():
            if _sha(archive.read(name)) != digests[name]:
                raise ValueError(f"bundled manifest changed: {name}")
    return reference


class CheckpointAttachments:
    """``store.log_artifacts(run_id, directory, artifact_path)`` receives each bundle once."""

    def __init__(self, store, state_path):
        self.store, self.state_path = store, Path(state_path)
        self.state = json.loads(self.state_path.read_text()) if self.state_path.exists() else {"attached": {}}

    def _candidates(self, root: Path) -> list[Path]:
        found = [p.parent for p in sorted((root / "checkpoints").glob("step-*/COMPLETE.json"))]
        return sorted(found, key=lambda p: int(p.name.split("-")[1]))

    def sync(self, spec: dict) -> dict:
        """``spec``: ``{"run_id", "root", "variant"}``."""
        root = Path(spec["root"])
        attached, skipped = [], []
        with SingleWriterLock(self.state_path.with_suffix(".lock")):
            if self.state_path.exists():                              # another instance may have attached checkpoints meanwhile
                self.state = json.loads(self.state_path.read_text())
            done = self.state["attached"].setdefault(spec["run_id"], {})
            for checkpoint in self._candidates(root):
                if checkpoint.name in done:
                    continue
                with tempfile.TemporaryDirectory() as scratch:
                    try:
                        reference = make_bundle(checkpoint, Path(scratch) / checkpoint.name, spec["variant"])
                    except (ValueError, KeyError, FileNotFoundError) as why:
                        skipped.append({"checkpoint": checkpoint.name, "reason": str(why)})
                        continue
                    self.store.log_artifacts(spec["run_id"], Path(scratch) / checkpoint.name, f"checkpoints/{checkpoint.name}")
                done[checkpoint.name] = {"marker_sha256": reference["checkpoint_marker_sha256"], "attached": time.time(), "source": str(checkpoint)}
                attached.append(checkpoint.name)
                atomic_write_json(self.state_path, self.state)
            catalog = {name: {**row, "source_available": Path(row["source"]).joinpath("COMPLETE.json").exists()} for name, row in done.items()}
            (root / "checkpoints").mkdir(parents=True, exist_ok=True)
            atomic_write_json(root / "checkpoints" / "CATALOG.json", {"run_id": spec["run_id"], "observed": time.time(), "checkpoints": catalog})
        return {"attached": attached, "skipped": skipped}


def log_artifacts_to_directory(store_root):
    """An artifact sink for ``FileTrackingStore``-style roots: copies the bundle under ``<root>/<run>/artifacts/``."""
    class _Sink:
        def log_artifacts(self, run_id, directory, artifact_path):
            target = Path(store_root) / run_id / "artifacts" / artifact_path
            if target.exists():
                raise FileExistsError(f"artifact already present: {artifact_path}")
            shutil.copytree(directory, target)
    return _Sink()
