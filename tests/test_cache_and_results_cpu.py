"""Content-addressed checkpoint staging and the metric-table rules."""
import hashlib
import json
import multiprocessing as mp

import pytest

from archlab_b200.ckpt import cache
from archlab_b200.services import results_table as rt


def _checkpoint(root):
    root.mkdir()
    files = {}
    for name, data in (("model.bin", b"m" * 1000), ("optim.bin", b"o" * 500)):
        (root / name).write_bytes(data)
        files[name] = hashlib.sha256(data).hexdigest()
    (root / "COMPLETE.json").write_text(json.dumps({"files": files, "step": 7}))
    return root


def _stage(args):
    src, dst = args
    return str(cache.stage_checkpoint(src, dst))


def test_concurrent_ranks_share_one_verified_copy(tmp_path):
    src = _checkpoint(tmp_path / "src")
    with mp.get_context("spawn").Pool(4) as pool:
        entries = set(pool.map(_stage, [(str(src), str(tmp_path / "cache"))] * 4))
    assert len(entries) == 1
    entry = next(iter(entries))
    assert (tmp_path / "cache").joinpath(entry).joinpath("VERIFIED.json").exists()
    assert sorted(p.name for p in (tmp_path / "cache").iterdir() if "partial" in p.name) == []
    assert (src / "model.bin").read_bytes() == b"m" * 1000                      # the source is untouched
    again = cache.stage_checkpoint(src, tmp_path / "cache")
    assert str(again) == entry
    (again / "model.bin").write_bytes(b"x" * 1000)                              # modified after verification
    with pytest.raises(ValueError, match="payload changed"):
        cache.stage_checkpoint(src, tmp_path / "cache")


def test_staging_refusals(tmp_path):
    src = _checkpoint(tmp_path / "src")
    (src / "optim.bin").write_bytes(b"tampered")
    with pytest.raises(ValueError, match="checksum mismatch"):
        cache.stage_checkpoint(src, tmp_path / "cache")
    assert [p for p in (tmp_path / "cache").iterdir() if p.is_dir()] == []      # nothing partial is left or published
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "COMPLETE.json").write_text(json.dumps({"files": {"../escape": "0" * 64}}))
    with pytest.raises(ValueError, match="unsafe payload name"):
        cache.stage_checkpoint(bad, tmp_path / "cache")


HEADER = ",".join(rt.REQUIRED)
GOOD = [HEADER, "c1,d12,matched,baseline,100,0.900000000,,3,1.0,complete,2026-01-02", "c1,d12,matched,kda,120,0.880000000,-0.020000000,3,0.9,complete,2026-01-02",
        "c1,d12,matched,broken,120,,,0,,failed-nonfinite,2026-01-02", "c2,d20,matched,baseline,500,0.8,,2,,partial,2026-01-03"]


def _table(tmp_path, lines):
    p = tmp_path / "metrics.csv"
    p.write_text("\n".join(lines) + "\n")
    return p


def test_metric_table_rules(tmp_path):
    assert rt.verify_table(_table(tmp_path, GOOD)) == {"rows": 4, "campaigns": 2}
    cases = {
        "paired delta disagrees": GOOD[:2] + ["c1,d12,matched,kda,120,0.88,-0.05,3,0.9,complete,2026-01-02"],
        "duplicate metric row": GOOD + [GOOD[1]],
        "unknown result status": GOOD[:2] + ["c1,d12,matched,x,1,0.9,,3,,done,2026-01-02"],
        "must contain 3 seeds": GOOD[:2] + ["c1,d12,matched,x,1,0.9,,2,,complete,2026-01-02"],
        "must not publish a BPB": GOOD[:2] + ["c1,d12,matched,x,1,0.9,,0,,failed-nonfinite,2026-01-02"],
        "invalid BPB": GOOD[:2] + ["c1,d12,matched,x,1,-0.9,,3,,complete,2026-01-02"],
        "invalid throughput ratio": GOOD[:2] + ["c1,d12,matched,x,1,0.9,,3,0,complete,2026-01-02"],
        "missing required columns": ["campaign,scale", "a,b"],
    }
    for message, lines in cases.items():
        with pytest.raises(ValueError, match=message):
            rt.verify_table(_table(tmp_path, lines))
    with pytest.raises(ValueError):
        rt.verify_table(_table(tmp_path, GOOD[:2] + ["c1,d12,matched,x,1,0.9,,3,,complete,not-a-date"]))
