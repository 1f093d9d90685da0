"""Executable-task index: contract validation, hash-ranked selection, digest-pinned images, offline verification."""
import json

import pytest

from archlab_b200.data import code_tasks as ct

IMAGE = "registry.example/tasks@sha256:" + "ab" * 32


def row(i, **edit):
    task = {"cwd": "/work", "docker_image": f"task-{i}:latest", "instance_id": f"task-{i}", "problem_statement": f"fix bug number {i}", "test_command": "pytest -q",
            "test_patch": f"diff {i}", "verifier_timeout_sec": 600, "dataset_type": "opensource-code"}
    task.update(edit)
    return {"data_source": "opensource-code", "ability": "swe", "prompt": [{"role": "user", "content": task["problem_statement"]}],
            "reward_model": {"style": "rule", "ground_truth": ""}, "extra_info": {"instance_id": task["instance_id"], "index": i, "instance_json": json.dumps(task)}}


def test_contract_and_selection():
    rows = [row(i) for i in range(20)]
    assert ct.validate_task(rows[3])["instance_id"] == "task-3"
    chosen = ct.select(rows, 6, 2, seed=7)
    assert len(chosen) == 8 and ct.select(list(reversed(rows)), 6, 2, seed=7) == chosen and ct.select(rows, 6, 2, seed=8) != chosen
    leak = row(1)
    leak["prompt"][0]["content"] += "\nhidden: diff 1"
    for bad, message in ((row(1, cwd="work"), "working directory"), (row(1, test_patch=""), "incomplete executable task"), (leak, "hidden test metadata"),
                         ({**row(1), "reward_model": {"style": "model"}}, "executable verifier"), ({**row(1), "ability": "math"}, "only software-engineering")):
        with pytest.raises(ValueError, match=message):
            ct.validate_task(bad)
    with pytest.raises(ValueError, match="duplicate"):
        ct.select(rows + [row(3)], 6, 2, seed=7)
    with pytest.raises(ValueError, match="insufficient"):
        ct.select(rows[:5], 6, 2, seed=7)
    with pytest.raises(ValueError, match="at most 128"):
        ct.select(rows, 120, 20, seed=7)
    with pytest.raises(ValueError, match="pinned by digest"):
        ct.bind_image(rows[0], "registry.example/tasks:latest")


def test_index_round_trip_and_tamper_detection(tmp_path):
    rows = [row(i) for i in range(20)]
    source = {"dataset": "example/tasks", "revision": "abc", "sha256": "0" * 64}
    manifest = ct.build_index(tmp_path / "idx", rows, lambda task: IMAGE, source=source, train=6, validation=2, seed=7)
    assert set(manifest["files"]) == {"index.jsonl", "train.jsonl", "validation.jsonl"}
    report = ct.verify_index(tmp_path / "idx" / "manifest.json", source=source)
    assert report["train"] == 6 and report["validation"] == 2
    train = [json.loads(l) for l in (tmp_path / "idx" / "train.jsonl").read_text().splitlines()]
    assert all(json.loads(r["extra_info"]["instance_json"])["docker_image"] == IMAGE for r in train)
    audit = ct.audit_prompt_lengths(tmp_path / "idx" / "manifest.json", lambda s: s.split(), prompt_limit=3)
    assert audit["prompts"] == 8 and audit["max_tokens"] == 4 and len(audit["over_limit"]) == 8
    with pytest.raises(FileExistsError):
        ct.build_index(tmp_path / "idx", rows, lambda task: IMAGE, source=source)
    with pytest.raises(ValueError, match="unexpected dataset source"):
        ct.verify_index(tmp_path / "idx" / "manifest.json", source={**source, "revision": "def"})
    lines = (tmp_path / "idx" / "train.jsonl").read_text().splitlines()
    (tmp_path / "idx" / "train.jsonl").write_text("\n".join(reversed(lines)) + "\n")
    with pytest.raises(ValueError, match="checksum mismatch"):
        ct.verify_index(tmp_path / "idx" / "manifest.json")
    eligible = {"selection_basis": "solved at least once by the reference agent", "instance_ids": [f"task-{i}" for i in range(10)]}
    ct.build_index(tmp_path / "idx2", rows, lambda task: IMAGE, source=source, train=6, validation=2, seed=7, eligibility=eligible)
    ct.verify_index(tmp_path / "idx2" / "manifest.json")
    with pytest.raises(ValueError, match="stated basis"):
        ct.build_index(tmp_path / "idx3", rows, lambda task: IMAGE, source=source, eligibility={"instance_ids": ["task-1"]})
