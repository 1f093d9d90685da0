"""Immutable evaluation checkpoints: links, milestones, catalogue."""
import json

import pytest
import torch

from archlab_b200.ckpt.formats import write_v41_sharded
from archlab_b200.services import eval_checkpoints as ec


def _save(path, tokens, budget=1000):
    state = {"w": torch.arange(8, dtype=torch.float32).view(4, 2)}
    write_v41_sharded(path, state, cursor={"step": tokens // 10, "supervised_tokens": tokens}, world_size=2, ep_size=2, expert_fsdp_size=1)
    marker = json.loads((path / "COMPLETE.json").read_text())
    marker["contract"]["target_supervised_tokens"] = budget
    (path / "COMPLETE.json").write_text(json.dumps(marker))
    for r in range(2):                                               # rank manifests must agree with the marker
        m = json.loads((path / f"rank-{r:02d}" / "MANIFEST.json").read_text())
        m["contract"] = marker["contract"]
        (path / f"rank-{r:02d}" / "MANIFEST.json").write_text(json.dumps(m))


def test_link_is_immutable_and_checked(tmp_path):
    bulk = (tmp_path / "bulk").resolve()
    bulk.mkdir()
    local = ec.link_checkpoint(tmp_path / "run" / "step-20", bulk / "step-20", accept_mount=lambda t: t == "fuse.bulk", mount_of=lambda p: "fuse.bulk")
    assert local.is_symlink() and local.resolve() == bulk / "step-20"
    with pytest.raises(FileExistsError):
        ec.link_checkpoint(tmp_path / "run" / "step-20", bulk / "step-21")
    with pytest.raises(FileExistsError):
        ec.link_checkpoint(tmp_path / "run" / "other", bulk / "step-20")
    with pytest.raises(ValueError, match="expected storage"):
        ec.link_checkpoint(tmp_path / "run" / "step-30", bulk / "step-30", accept_mount=lambda t: t == "fuse.bulk", mount_of=lambda p: "ext4")
    with pytest.raises(ValueError, match="absolute path"):
        ec.link_checkpoint(tmp_path / "run" / "step-40", "relative/step-40")
    assert isinstance(ec.mount_type(tmp_path), str)


def test_catalogue_accepts_only_declared_verified_milestones(tmp_path):
    bulk = (tmp_path / "bulk").resolve()
    bulk.mkdir()
    out = tmp_path / "run"
    out.mkdir()
    link = ec.link_checkpoint(out / "step-40", bulk / "step-40")
    _save(link, tokens=410)
    assert ec.milestones(1000) == [200, 400, 600, 800, 1000]
    receipt = ec.record_evaluation_checkpoint(out, link, milestone=400, budget=1000)
    assert receipt["ranks"] == 2
    catalogue = json.loads((out / "EVAL_CHECKPOINTS.json").read_text())
    assert catalogue["checkpoints"][0]["milestone_tokens"] == 400 and catalogue["checkpoints"][0]["bulk_path"] == str(bulk / "step-40")
    for kwargs, message in (({"milestone": 400, "budget": 1000}, "duplicate"), ({"milestone": 500, "budget": 1000}, "outside the declared milestones"),
                            ({"milestone": 600, "budget": 1000}, "predates"), ({"milestone": 400, "budget": 2000}, "budget differs")):
        with pytest.raises(ValueError, match=message):
            ec.record_evaluation_checkpoint(out, link, **kwargs)
    plain = out / "not-a-link"
    _save(plain, tokens=800)
    with pytest.raises(ValueError, match="must be a link"):
        ec.record_evaluation_checkpoint(out, plain, milestone=800, budget=1000)
    assert ec.on_rank_zero(lambda: 7) == 7                            # without a process group: runs in place
