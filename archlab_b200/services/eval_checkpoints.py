"""Immutable evaluation checkpoints: written through a local link into bulk storage and catalogued at declared token
milestones.

* ``link_checkpoint(local, target)``: checkpoint names are immutable, so neither side may exist; the target must be an
  absolute path without symlinks and (when a mount check is supplied) must live on the expected kind of mount
  (``mount_type`` reads ``findmnt``); the target directory is created and ``local`` becomes a symlink to it, so the
  trainer writes "locally" and the bytes land in bulk storage.
* ``on_rank_zero(fn)``: rank 0 runs ``fn`` and every rank receives its value or raises its error, so a refused link or
  record stops all ranks together.
* ``record_evaluation_checkpoint``: a checkpoint may enter ``EVAL_CHECKPOINTS.json`` only at one of the declared
  milestones of its token budget (fifths by default), only once per milestone, only if it verifies structurally
  (``services.retention.verify_sharded``), belongs to a run with that budget and has really reached the milestone.
(The reference does this for its object-storage mount: src/archlab/storage/oss_checkpoint.py:13-100.)
"""
from __future__ import annotations

import json
import subprocess
from pathlib import Path
from typing import Callable

from ..contracts.substrate import atomic_write_json
from .retention import verify_sharded


def mount_type(path: Path) -> str:
    """File-system type of the mount that holds ``path`` (or its nearest existing parent)."""
    probe = Path(path)
    while not probe.exists():
        probe = probe.parent
    out = subprocess.check_output(["findmnt", "--json", "--target", str(probe), "--output", "TARGET,FSTYPE"], text=True)
    return json.loads(out)["filesystems"][0]["fstype"]


def link_checkpoint(local, target, *, accept_mount: Callable[[str], bool] | None = None, mount_of: Callable[[Path], str] = mount_type) -> Path:
    local, target = Path(local), Path(target)
    if not target.is_absolute() or target.resolve() != target:
        raise ValueError("the bulk destination must be an absolute path without symlinks")
    if local.exists() or local.is_symlink() or target.exists():
        raise FileExistsError("checkpoint names are immutable; refusing to overwrite")
    if accept_mount is not None and not accept_mount(mount_of(target)):
        raise ValueError(f"checkpoint destination is not on the expected storage: {target}")
    target.mkdir(parents=True, exist_ok=False)
    local.parent.mkdir(parents=True, exist_ok=True)
    local.symlink_to(target, target_is_directory=True)
    return local


def on_rank_zero(function: Callable[[], object], group=None):
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return function()
    box = [None]
    if dist.get_rank(group) == 0:
        try:
            box[0] = {"value": function()}
        except Exception as error:                               # travels to every rank
            box[0] = {"error": f"{type(error).__name__}: {error}"}
    dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    if "error" in box[0]:
        raise RuntimeError(box[0]["error"])
    return box[0]["value"]


def milestones(budget: int, parts: int = 5) -> list[int]:
    if budget <= 0 or budget % parts:
        raise ValueError("the token budget must be a positive multiple of the number of milestones")
    return [budget // parts * i for i in range(1, parts + 1)]


def record_evaluation_checkpoint(output, checkpoint, *, milestone: int, budget: int, parts: int = 5,
                                 accept_mount: Callable[[str], bool] | None = None, mount_of: Callable[[Path], str] = mount_type,
                                 verify: Callable[[Path], dict] = verify_sharded) -> dict:
    output, checkpoint = Path(output), Path(checkpoint)
    if milestone not in milestones(budget, parts):
        raise ValueError("evaluation checkpoint is outside the declared milestones")
    if not checkpoint.is_symlink():
        raise ValueError("an evaluation checkpoint must be a link into bulk storage")
    target = checkpoint.resolve(strict=True)
    if accept_mount is not None and not accept_mount(mount_of(target)):
        raise ValueError(f"checkpoint destination is not on the expected storage: {target}")
    receipt = verify(target)
    marker = json.loads((target / "COMPLETE.json").read_text())
    if marker.get("contract", {}).get("target_supervised_tokens", budget) != budget:
        raise ValueError("checkpoint training budget differs from its milestone schedule")
    if marker["cursor"]["supervised_tokens"] < milestone:
        raise ValueError("checkpoint predates its token milestone")
    catalogue_path = output / "EVAL_CHECKPOINTS.json"
    catalogue = json.loads(catalogue_path.read_text()) if catalogue_path.exists() else {"checkpoints": []}
    if any(row["milestone_tokens"] == milestone for row in catalogue["checkpoints"]):
        raise ValueError("duplicate evaluation checkpoint milestone")
    catalogue["checkpoints"].append({"milestone_tokens": milestone, "path": str(checkpoint), "bulk_path": str(target),
                                     "cursor": marker["cursor"], "verification": receipt})
    catalogue["checkpoints"].sort(key=lambda row: row["milestone_tokens"])
    atomic_write_json(catalogue_path, catalogue)
    return receipt
