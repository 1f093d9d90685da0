"""Does a public benchmark overlap with what the model was actually trained on?  A bounded audit over this framework's
own data lineage: RL problem sets and prepared corpora.

Two matching rules, both stated in the report: the exact hash of the NFC / whitespace-normalised problem, and the
benchmark question's format-normalised text (lower case, letters, digits and arithmetic signs only, ``\\left`` / ``\\right``
dropped) contained in the training prompt.  Signs are kept: a benchmark about -3 is not the same as one about +3.

* ``audit_rl(cases, problem_set_dir)`` checks ``train.jsonl`` and ``heldout.jsonl`` of an RL problem set (file hashes
  verified against its manifest first).
* ``audit_prepared(cases, corpus_root, tokens_read, ...)`` walks the sealed per-document metadata of a prepared corpus
  (``problem_sha256`` per document; every sidecar's size and hash are checked against its part's READY marker), finds the
  retained documents that match a benchmark problem, and says which of them the run had READ by a given token cursor.
  The cursor is rounded UP to whole global batches: a partly used last batch counts as exposed.
The audit cannot rule out paraphrases or contamination of a base model's pre-training, and the report says so.
(Reference: src/archlab/evaluation/limite_math_overlap.py:23-140.)
"""
from __future__ import annotations

import gzip
import json
import math
import re
import unicodedata
from pathlib import Path

from ..contracts.substrate import sha256_file
from ..data.rl_problems import problem_key

LIMITATION = "exact and format-normalised matching only; paraphrases and undisclosed pre-training cannot be excluded"


def normalized_text(text: str) -> str:
    text = unicodedata.normalize("NFC", text).lower().replace("\u2212", "-")
    text = re.sub(r"\\(?:left|right)\b", "", text)
    return "".join(re.findall(r"[a-z0-9]+|[+-]", text))


def _prompt_text(row: dict) -> str:
    prompt = row["prompt"]
    return prompt if isinstance(prompt, str) else " ".join(m.get("content", "") for m in prompt)


def audit_rl(cases: list[dict], data) -> dict:
    data = Path(data)
    manifest = json.loads((data / "manifest.json").read_text())
    matches, counts, files = [], {}, {}
    targets = [(c, problem_key(c["question"]), normalized_text(c["question"])) for c in cases]
    for split in ("train", "heldout"):
        path = data / f"{split}.jsonl"
        files[split] = sha256_file(path)
        if files[split] != manifest["files"][split]["sha256"]:
            raise ValueError(f"the problem set changed after it was sealed: {split}")
        rows = [json.loads(line) for line in path.read_text().splitlines() if line.strip()]
        counts[split] = len(rows)
        for row in rows:
            prompt = normalized_text(_prompt_text(row))
            for case, key, text in targets:
                exact = row.get("problem_sha256") == key
                if exact or (text and text in prompt):
                    matches.append({"problem_id": case["id"], "split": split, "uuid": row.get("uuid"),
                                    "method": "exact normalised-whitespace hash" if exact else "format-normalised question contained in the prompt"})
    return {"rows": counts, "matches": matches, "files": files, "manifest_sha256": sha256_file(data / "manifest.json")}


def audit_prepared(cases: list[dict], corpus_root, *, tokens_read: int, context: int, global_windows_per_step: int, partition: str = "train",
                   task_order: list[str] | None = None) -> dict:
    """Documents are read in ``task_order`` (default: the contract's task order), back to back; a document counts as read
    when its first token lies before the (rounded-up) cursor."""
    root = Path(corpus_root)
    contract = json.loads((root / "manifest.json").read_text())
    hashes = {problem_key(c["question"]): c for c in cases}
    cursor_tokens = math.ceil(tokens_read / (context * global_windows_per_step)) * global_windows_per_step * context
    retained, seen, offset, documents = [], [], 0, 0
    for task_id in task_order or [t["id"] for t in contract["tasks"]]:
        part = root / "parts" / task_id
        ready = json.loads((part / "READY.json").read_text())
        name = ready["partitions"][partition]["prefix"] + ".metadata.jsonl.gz"
        expected = next(f for f in ready["files"] if f["name"] == name)
        sidecar = part / name
        if sidecar.stat().st_size != expected["bytes"] or sha256_file(sidecar) != expected["sha256"]:
            raise ValueError(f"sealed document metadata changed: {task_id}")
        with gzip.open(sidecar, "rt") as f:
            for line in f:
                row = json.loads(line)
                documents += 1
                case = hashes.get(row.get("problem_sha256"))
                if case is not None:
                    entry = {"problem_id": case["id"], "task": task_id, "source_row": row["row"], "document_tokens": row["tokens"],
                             "first_token_offset": offset, "method": "exact sealed problem hash", "read_by_cursor": offset < cursor_tokens}
                    retained.append(entry)
                    if entry["read_by_cursor"]:
                        seen.append(entry)
                offset += row["tokens"]
    return {"documents_scanned": documents, "retained_document_matches": retained, "seen_by_cursor": seen,
            "seen_problem_ids": sorted({e["problem_id"] for e in seen}), "tokens_read": tokens_read, "cursor_tokens": cursor_tokens,
            "cursor_rule": "rounded up to whole global batches; a partly used final batch counts as exposed",
            "contract_sha256": sha256_file(root / "manifest.json")}


def audit(cases_file, *, rl_data=None, prepared=None, **prepared_kw) -> dict:
    cases = [json.loads(line) for line in Path(cases_file).read_text().splitlines() if line.strip()]
    if len({c["id"] for c in cases}) != len(cases):
        raise ValueError("benchmark case ids must be unique")
    report = {"format": "archlab-benchmark-overlap-audit-v1", "cases": len(cases), "cases_sha256": sha256_file(cases_file), "limitation": LIMITATION}
    if rl_data is not None:
        report["rl"] = audit_rl(cases, rl_data)
    if prepared is not None:
        report["prepared"] = audit_prepared(cases, prepared, **prepared_kw)
    return report
