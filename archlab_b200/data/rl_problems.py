"""Problem sets for verifier-based RL: nothing the policy has already seen, one label per problem, split after
de-duplication.

The rules (the reference's math-RL data preparation, src/archlab/rl/nemotron_data.py:30-262):

* a problem is identified by the SHA-256 of its NFC-normalised, whitespace-collapsed text (``problem_key``);
* an *exposure set* (problem keys and source ids that earlier SFT / pilot corpora contained) removes problems the policy
  may have been trained on; it is built from the metadata sidecars of prepared corpora, never from model-visible text;
* de-duplication happens *before* the train / held-out split, so a duplicate can never sit on both sides;
* a problem whose duplicates disagree on the canonical gold answer, or carry a gold the verifier cannot canonicalise, is
  dropped entirely (keeping one of two disagreeing labels would silently choose it); so is every problem whose source id
  also appears with a different text;
* the surviving problems are ordered by a seeded hash of their key, the held-out set is the head of that order, the
  training set follows it: adding rows to the input does not reshuffle earlier choices;
* every drop is counted by reason.
"""
from __future__ import annotations

import hashlib
import json
import unicodedata
from collections import Counter, defaultdict
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Iterable


def problem_key(problem: str) -> str:
    if not isinstance(problem, str) or not problem.strip():
        raise ValueError("a nonempty problem is required")
    return hashlib.sha256(" ".join(unicodedata.normalize("NFC", problem).split()).encode()).hexdigest()


@dataclass
class Exposure:
    """What earlier training already contained."""
    problem_hashes: set[str] = field(default_factory=set)
    source_ids: set[str] = field(default_factory=set)
    artifacts: list[dict] = field(default_factory=list)          # (path, sha256) of every file the set was built from

    def add_metadata(self, path, *, text_field: str = "problem", id_field: str = "uuid") -> "Exposure":
        """One JSONL (optionally gzip) sidecar with a row per document; rows without the text field are skipped."""
        import gzip

        path = Path(path)
        raw = path.read_bytes()
        self.artifacts.append({"path": str(path.resolve()), "sha256": hashlib.sha256(raw).hexdigest()})
        text = gzip.decompress(raw).decode() if path.suffix == ".gz" else raw.decode()
        for line in filter(None, map(str.strip, text.splitlines())):
            row = json.loads(line)
            if isinstance(row.get(text_field), str) and row[text_field].strip():
                self.problem_hashes.add(problem_key(row[text_field]))
            if row.get("problem_sha256"):
                self.problem_hashes.add(row["problem_sha256"])
            if row.get(id_field):
                self.source_ids.add(str(row[id_field]))
        return self

    def seen(self, key: str, source_id: str) -> bool:
        return key in self.problem_hashes or bool(source_id and source_id in self.source_ids)


def select_problems(rows: Iterable[dict], exposure: Exposure, *, train_size: int, heldout_size: int, seed: int,
                    canonicalizer: Callable[[str], str | None], max_problem_chars: int = 6000, tag: str = "rl-problems"):
    """-> (train records, held-out records, counts by reason).  ``rows`` carry ``problem``, ``expected_answer``, an
    optional ``uuid`` and ``_source = {"file": ..., "row": ...}`` (the earliest source wins among duplicates)."""
    if min(train_size, heldout_size) < 1:
        raise ValueError("train and held-out sizes must be positive")
    counts: Counter = Counter()
    best: dict[str, dict] = {}
    golds: dict[str, set] = defaultdict(set)
    texts_of_id: dict[str, set] = defaultdict(set)
    order = lambda rec: (rec["source"].get("file", ""), rec["source"].get("row", 0))
    for row in rows:
        counts["scanned_rows"] += 1
        problem = row.get("problem")
        if not isinstance(problem, str) or not problem.strip() or len(problem) > max_problem_chars:
            counts["invalid_or_long_problem"] += 1
            continue
        key, source_id = problem_key(problem), str(row.get("uuid") or "")
        if exposure.seen(key, source_id):
            counts["previously_exposed_problem_or_id"] += 1
            continue
        if source_id:
            texts_of_id[source_id].add(key)
        gold = row.get("expected_answer")
        canonical = canonicalizer(gold) if isinstance(gold, str) else None
        golds[key].add(canonical)                                   # None poisons the problem too
        if canonical is None:
            counts["unsupported_gold"] += 1
            continue
        record = {"id": key, "problem_sha256": key, "uuid": source_id, "prompt": [{"role": "user", "content": problem}],
                  "expected_answer": gold, "canonical_answer": canonical, "source": dict(row.get("_source") or {})}
        if key not in best or order(record) < order(best[key]):
            best[key] = record
    aliased = {key for keys in texts_of_id.values() if len(keys) > 1 for key in keys}
    clean = [rec for key, rec in best.items() if len(golds[key]) == 1 and key not in aliased]
    counts["conflicting_or_aliased_problems"] = len(best) - len(clean)
    counts["eligible_unique_problems"] = len(clean)
    clean.sort(key=lambda rec: hashlib.sha256(f"{tag}:{seed}:{rec['id']}".encode()).digest())
    if len(clean) < train_size + heldout_size:
        raise ValueError(f"only {len(clean)} eligible unique problems; need {train_size + heldout_size}; {dict(counts)}")
    return clean[heldout_size:heldout_size + train_size], clean[:heldout_size], dict(counts)


def write_problem_set(out_dir, train: list[dict], heldout: list[dict], counts: dict, exposure: Exposure, *, seed: int) -> dict:
    """``train.jsonl``, ``heldout.jsonl`` and a manifest that pins their hashes, the counts and the exposure artifacts."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=False)
    files = {}
    for name, records in (("train", train), ("heldout", heldout)):
        body = "".join(json.dumps(r, sort_keys=True, ensure_ascii=False) + "\n" for r in records).encode()
        (out / f"{name}.jsonl").write_bytes(body)
        files[name] = {"records": len(records), "sha256": hashlib.sha256(body).hexdigest()}
    if {r["id"] for r in train} & {r["id"] for r in heldout}:
        raise AssertionError("a problem sits on both sides of the split")
    manifest = {"format": "archlab-rl-problem-set-v1", "seed": seed, "files": files, "counts": counts,
                "exposure": {"problem_hashes": len(exposure.problem_hashes), "source_ids": len(exposure.source_ids),
                             "artifacts": exposure.artifacts}}
    (out / "manifest.json").write_text(json.dumps(manifest, indent=1, sort_keys=True) + "\n")
    return manifest
