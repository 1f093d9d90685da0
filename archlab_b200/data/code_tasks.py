"""A bounded, reproducible index of executable software-engineering tasks for agentic RL.

Tasks come as rows whose ``extra_info.instance_json`` holds the executable contract (working directory, container
image, problem statement, hidden test patch and command, verifier timeout).  The index keeps task JSON intact; the only
transformation pins each task's container image to an immutable digest through a caller-supplied ``resolve_image``
(there is no network access in this module).  Hidden tests never reach the prompt: the prompt must be exactly the
problem statement, and the reward must be the executable verifier's.

* ``validate_task(row)``  the contract above, without executing anything;
* ``select(rows, train, validation, seed)``  hash-ranks unique tasks (``sha256(seed NUL instance_id)``), independent of
  the source order; duplicates by identity or by prompt are an error, not silently dropped;
* ``build_index(...)``  writes ``train.jsonl`` / ``validation.jsonl`` (rows with pinned images), ``index.jsonl`` (digests of
  prompt, source JSON and test patch per task) and ``manifest.json`` (source hash, selection rule, file hashes); refuses
  a non-empty output directory;
* ``verify_index(manifest)``  re-derives all of it offline: file hashes, split sizes, index entries, image pinning and the
  deterministic selection itself;
* ``audit_prompt_lengths``  token counts of the immutable prompts against a limit, with an injected tokenizer.
(Reference: src/archlab/data/mimo_code.py:36-320.)
"""
from __future__ import annotations

import copy
import hashlib
import json
import re
from pathlib import Path
from typing import Callable

REQUIRED = ("cwd", "docker_image", "instance_id", "problem_statement", "test_command", "test_patch", "verifier_timeout_sec")
PINNED_IMAGE = re.compile(r"[\w./-]+@sha256:[0-9a-f]{64}")
TOTAL_LIMIT = 128


def digest(value: bytes) -> str:
    return hashlib.sha256(value).hexdigest()


def validate_task(row: dict, *, data_source: str = "opensource-code", ability: str = "swe") -> dict:
    task = json.loads(row["extra_info"]["instance_json"])
    if row.get("data_source") != data_source or row.get("ability") != ability or task.get("dataset_type") != data_source:
        raise ValueError("only software-engineering agent tasks of the declared source are permitted")
    if any(not task.get(k) for k in REQUIRED):
        raise ValueError("incomplete executable task: environment or test metadata missing")
    if row["extra_info"].get("instance_id") != task["instance_id"]:
        raise ValueError("task identity mismatch")
    if not task["cwd"].startswith("/") or int(task["verifier_timeout_sec"]) <= 0:
        raise ValueError("invalid sandbox working directory or verifier timeout")
    if row.get("prompt") != [{"role": "user", "content": task["problem_statement"]}]:
        raise ValueError("unexpected prompt; hidden test metadata must stay outside the prompt")
    if row.get("reward_model") != {"style": "rule", "ground_truth": ""}:
        raise ValueError("rewards must come from the executable verifier")
    return task


def select(rows: list[dict], train: int, validation: int, seed: int) -> list[dict]:
    if train < 1 or validation < 1 or train + validation > TOTAL_LIMIT:
        raise ValueError(f"positive train / validation counts, at most {TOTAL_LIMIT} in total")
    ids, prompts, ranked = set(), set(), []
    for row in rows:
        task = validate_task(row)
        key, prompt = task["instance_id"], digest(task["problem_statement"].encode())
        if key in ids or prompt in prompts:
            raise ValueError("duplicate task identity or prompt; resolve before splitting")
        ids.add(key), prompts.add(prompt)
        ranked.append((digest(f"{seed}\0{key}".encode()), key, row))
    if len(ranked) < train + validation:
        raise ValueError("insufficient unique tasks")
    return [row for _, _, row in sorted(ranked, key=lambda t: t[:2])[:train + validation]]


def bind_image(row: dict, resolved_image: str) -> dict:
    if not PINNED_IMAGE.fullmatch(resolved_image):
        raise ValueError("a task image must be pinned by digest")
    out = copy.deepcopy(row)
    task = validate_task(out)
    task["docker_image"] = resolved_image
    out["extra_info"]["instance_json"] = json.dumps(task, ensure_ascii=False, sort_keys=True)
    return out


def _write_jsonl(path: Path, rows) -> None:
    path.write_text("".join(json.dumps(r, sort_keys=True, ensure_ascii=False) + "\n" for r in rows))


def build_index(output, rows: list[dict], resolve_image: Callable[[dict], str], *, source: dict, train: int = 64, validation: int = 8,
                seed: int = 42, eligibility: dict | None = None) -> dict:
    """``source``: provenance of ``rows`` (dataset, revision, sha256 ...), copied into the manifest.  ``eligibility``:
    ``{"selection_basis": str, "instance_ids": [...]}`` restricts the candidates to a stated, unique list."""
    output = Path(output)
    if output.exists() and any(output.iterdir()):
        raise FileExistsError(f"refusing to overwrite a dataset index: {output}")
    if eligibility is not None:
        ids = eligibility.get("instance_ids") or []
        if not eligibility.get("selection_basis") or not ids or len(set(ids)) != len(ids):
            raise ValueError("candidate selection needs a stated basis and unique task identities")
        rows = [r for r in rows if validate_task(r)["instance_id"] in set(ids)]
        if len(rows) != len(ids):
            raise ValueError("candidate identities are missing from the source")
    chosen = select(rows, train, validation, seed)
    bound = [bind_image(r, resolve_image(validate_task(r))) for r in chosen]
    output.mkdir(parents=True, exist_ok=True)
    index = []
    for i, (row, pinned) in enumerate(zip(chosen, bound)):
        task = validate_task(row)
        index.append({"split": "train" if i < train else "validation", "instance_id": task["instance_id"], "source_index": row["extra_info"].get("index"),
                      "prompt_sha256": digest(task["problem_statement"].encode()), "source_instance_sha256": digest(row["extra_info"]["instance_json"].encode()),
                      "test_patch_sha256": digest(task["test_patch"].encode()), "cwd": task["cwd"], "test_command": task["test_command"],
                      "verifier_timeout_sec": task["verifier_timeout_sec"], "source_image": task["docker_image"],
                      "resolved_image": validate_task(pinned)["docker_image"]})
    _write_jsonl(output / "index.jsonl", index)
    _write_jsonl(output / "train.jsonl", bound[:train])
    _write_jsonl(output / "validation.jsonl", bound[train:])
    selection = {"method": "sha256(seed + NUL + instance_id)", "seed": seed, "train": train, "validation": validation, "total_limit": TOTAL_LIMIT}
    if eligibility is not None:
        selection["eligibility"] = eligibility
    manifest = {"schema_version": 1, "source": source, "selection": selection,
                "transformations": ["container image alias resolved to an immutable digest"],
                "tokenization": "deferred to the multi-turn runner; no truncation or text-only conversion",
                "qualification": "index_only: image execution and policy trajectories still require qualification",
                "files": {p.name: {"sha256": digest(p.read_bytes()), "bytes": p.stat().st_size} for p in sorted(output.iterdir()) if p.is_file()}}
    (output / "manifest.json").write_text(json.dumps(manifest, indent=2, sort_keys=True) + "\n")
    return manifest


def _read_jsonl(path: Path) -> list[dict]:
    return [json.loads(line) for line in path.read_text().splitlines() if line.strip()]


def verify_index(manifest_path, *, source: dict | None = None) -> dict:
    manifest_path = Path(manifest_path)
    manifest, root = json.loads(manifest_path.read_text()), manifest_path.parent
    if source is not None and manifest.get("source") != source:
        raise ValueError("unexpected dataset source or revision")
    if set(manifest["files"]) != {"train.jsonl", "validation.jsonl", "index.jsonl"}:
        raise ValueError("the payload catalogue is incomplete or unexpected")
    for name, meta in manifest["files"].items():
        payload = (root / name).read_bytes()
        if len(payload) != meta["bytes"] or digest(payload) != meta["sha256"]:
            raise ValueError(f"dataset checksum mismatch: {name}")
    sel = manifest["selection"]
    allowed = None
    if "eligibility" in sel:
        allowed = sel["eligibility"]["instance_ids"]
        if not sel["eligibility"].get("selection_basis") or not allowed or len(set(allowed)) != len(allowed):
            raise ValueError("invalid candidate eligibility contract")
    rows = []
    for split in ("train", "validation"):
        part = _read_jsonl(root / f"{split}.jsonl")
        if len(part) != sel[split]:
            raise ValueError(f"dataset split count mismatch: {split}")
        rows += part
    index = _read_jsonl(root / "index.jsonl")
    if len(index) != len(rows):
        raise ValueError("dataset index count mismatch")
    for i, (row, entry) in enumerate(zip(rows, index)):
        task = validate_task(row)
        if allowed is not None and task["instance_id"] not in allowed:
            raise ValueError("a selected task is outside the declared candidate set")
        want = {"instance_id": task["instance_id"], "split": "train" if i < sel["train"] else "validation",
                "prompt_sha256": digest(task["problem_statement"].encode()), "test_patch_sha256": digest(task["test_patch"].encode()),
                "resolved_image": task["docker_image"]}
        if any(entry.get(k) != v for k, v in want.items()):
            raise ValueError("the dataset index disagrees with the task payload")
        if not PINNED_IMAGE.fullmatch(task["docker_image"]):
            raise ValueError("a task image is not pinned by digest")
    if select(rows, sel["train"], sel["validation"], sel["seed"]) != rows:
        raise ValueError("task partition or order disagrees with the deterministic selection")
    return {"train": sel["train"], "validation": sel["validation"], "manifest_sha256": digest(manifest_path.read_bytes()),
            "qualification": "data_index_verified; sandbox and policy trajectory not evaluated"}


def audit_prompt_lengths(manifest_path, encode: Callable[[str], list[int]], prompt_limit: int) -> dict:
    root = Path(manifest_path).parent
    lengths = {}
    for split in ("train", "validation"):
        for row in _read_jsonl(root / f"{split}.jsonl"):
            task = validate_task(row)
            lengths[task["instance_id"]] = len(encode(task["problem_statement"]))
    over = sorted(k for k, n in lengths.items() if n > prompt_limit)
    return {"prompts": len(lengths), "max_tokens": max(lengths.values()), "limit": prompt_limit, "over_limit": over,
            "note": "prompts are immutable inputs; generated tokens belong to rollout telemetry"}
