"""Task-parallel corpus preparation: READY parts, resume, verified reuse, finalisation."""
import json

import numpy as np
import pytest

from archlab_b200.data import prepare_job as pj


class ByteTok:
    def encode(self, text):
        return list(text.encode())


ROWS = [{"id": f"g{i % 7}", "text": f"document number {i}", "keep": i % 5 != 0} for i in range(40)]
TASKS = [{"id": "t0", "source": "toy.jsonl", "row_start": 0, "rows": 25}, {"id": "t1", "source": "toy.jsonl", "row_start": 25, "rows": 15}]
render = lambda row: row["text"] if row["keep"] else None


def _contract(root, **extra):
    return pj.Contract.create(root, tokenizer_sha256="tok", renderer_sha256="r1", tasks=TASKS, heldout_fraction=0.3, split_seed=3, extra=extra)


def _run(root, task):
    rows = ROWS[task["row_start"]:task["row_start"] + task["rows"]]
    return pj.run_task(root, task["id"], iter(rows), render, ByteTok(), eod=0)


def test_tasks_publish_verified_parts_and_finalise(tmp_path):
    root = tmp_path / "v1"
    _contract(root)
    with pytest.raises(ValueError, match="tasks without a part"):
        pj.finalise(root)
    ready = [_run(root, t) for t in TASKS]
    assert ready[0]["documents"] + ready[0]["excluded_documents"] == 25 and ready[0]["excluded_documents"] == 5
    assert not list((root / ".scratch").iterdir())                          # published by rename, nothing left behind
    done = pj.finalise(root)
    total_docs = done["partitions"]["train"]["documents"] + done["partitions"]["heldout"]["documents"]
    assert total_docs == 32 and done["excluded_documents"] == 8 and done["partitions"]["heldout"]["documents"] > 0
    docs = pj.read_partition(root, "t0", "train") + pj.read_partition(root, "t0", "heldout")
    texts = sorted(bytes(d[:-1].astype(np.uint8)).decode() for d in docs)
    assert texts == sorted(r["text"] for r in ROWS[:25] if r["keep"]) and all(d[-1] == 0 for d in docs)
    # groups never straddle the split
    meta = lambda part: [json.loads(l)["row"] for l in __import__("gzip").open(root / "parts" / "t0" / f"t0-{part}.metadata.jsonl.gz", "rt")]
    assert not {ROWS[r]["id"] for r in meta("train")} & {ROWS[r]["id"] for r in meta("heldout")}
    # a second call finds the part and does not recompute
    assert _run(root, TASKS[0]) == ready[0]


def test_refusals_and_damage(tmp_path):
    root = tmp_path / "v1"
    _contract(root)
    with pytest.raises(ValueError, match="different dataset contract"):
        pj.Contract.create(root, tokenizer_sha256="other", renderer_sha256="r1", tasks=TASKS)
    with pytest.raises(ValueError, match="expected 25 rows"):
        pj.run_task(root, "t0", iter(ROWS[:10]), render, ByteTok(), eod=0)
    assert not (root / "parts" / "t0").exists()
    _run(root, TASKS[0])
    victim = root / "parts" / "t0" / "t0-train.bin"
    victim.write_bytes(victim.read_bytes()[:-4])
    with pytest.raises(ValueError, match="payload changed"):
        _run(root, TASKS[0])
    with pytest.raises(ValueError, match="unique ids"):
        pj.Contract.create(tmp_path / "bad", tokenizer_sha256="t", renderer_sha256="r", tasks=[TASKS[0], TASKS[0]])


def test_reuse_of_an_earlier_version(tmp_path):
    old, new = tmp_path / "v1", tmp_path / "v2"
    _contract(old, schema_version=1)
    _run(old, TASKS[0])
    _contract(new, schema_version=2)
    with pytest.raises(ValueError, match="more than the declared keys"):
        pj.reuse_parts(new, old, harmless_keys=set())
    out = pj.reuse_parts(new, old, harmless_keys={"schema_version"})
    assert out == {"adopted": ["t0"], "skipped": []}
    ready = json.loads((new / "parts" / "t0" / "READY.json").read_text())
    assert ready["contract_sha256"] == pj.Contract.load(new).sha256 and ready["reused_from"]["contract_sha256"] == pj.Contract.load(old).sha256
    assert (new / "parts" / "t0" / "ORIGIN_READY.json").exists()
    _run(new, TASKS[1])
    assert pj.finalise(new)["partitions"]["train"]["documents"] > 0
    # a damaged earlier part is skipped with its reason, not adopted
    third = tmp_path / "v3"
    _contract(third, schema_version=3)
    (old / "parts" / "t0" / "t0-train.idx").write_bytes(b"")
    out = pj.reuse_parts(third, old, harmless_keys={"schema_version"})
    assert out["adopted"] == [] and "payload changed" in out["skipped"][0]["reason"]
