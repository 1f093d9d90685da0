"""Corpus preparation: documents -> token parts with a completion marker, and the filters in front of it.

* ``prepare_token_parts``  - tokenise documents (each followed by an end-of-document token), cut the stream into
                             raw int32 parts of a fixed token count, write them atomically and finish with
                             ``DATA_READY.json`` (part list with sizes and SHA-256, tokenizer identity, token
                             count): a reader that finds the marker can trust every part
                             (the reference's ``megatron/data.py`` parquet/bin -> raw-int32 parts + DATA_READY.json).
* ``verify_token_parts``   - re-hash against the marker.
* ``normalise_math_record``/ ``filter_math_records`` - the Nemotron-style math pipeline's admission rules: a
                             record needs a problem, a final answer that canonicalises, a bounded length, and
                             must not duplicate an earlier problem after whitespace / case folding
                             (src/archlab/preprocessing/nemotron_math.py).
* ``split_by_group``       - deterministic held-out split by a stable hash of a group id (documents of one
                             group never land on both sides).
"""
from __future__ import annotations

import hashlib
import json
import os
import re
from pathlib import Path
from typing import Iterable

import numpy as np

from ..services.rewards import canonical_math_answer

FORMAT = "archlab-token-parts-v1"


def _atomic_bytes(path: Path, data: bytes) -> None:
    tmp = path.with_name(f".{path.name}.tmp")
    with open(tmp, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def prepare_token_parts(documents: Iterable[str], tokenizer, out_dir: Path, *, part_tokens: int, eod: int,
                        tokenizer_sha256: str | None = None) -> dict:
    out = Path(out_dir)
    if (out / "DATA_READY.json").exists():
        raise FileExistsError("output already holds a finished dataset")
    out.mkdir(parents=True, exist_ok=True)
    parts, buf, total, docs = [], [], 0, 0

    def flush(final: bool):
        nonlocal buf
        while len(buf) >= part_tokens or (final and buf):
            chunk, buf = buf[:part_tokens], buf[part_tokens:]
            arr = np.asarray(chunk, dtype=np.int32)
            name = f"part-{len(parts):05d}.bin"
            _atomic_bytes(out / name, arr.tobytes())
            parts.append({"file": name, "tokens": int(arr.size), "sha256": hashlib.sha256(arr.tobytes()).hexdigest()})

    for doc in documents:
        ids = tokenizer.encode(doc)
        buf.extend(ids)
        buf.append(eod)
        total += len(ids) + 1
        docs += 1
        flush(False)
    flush(True)
    marker = {"format": FORMAT, "dtype": "int32", "parts": parts, "tokens": total, "documents": docs, "end_of_document": eod,
              "tokenizer_sha256": tokenizer_sha256 or (tokenizer.sha256() if hasattr(tokenizer, "sha256") else None)}
    _atomic_bytes(out / "DATA_READY.json", (json.dumps(marker, indent=1, sort_keys=True) + "\n").encode())
    return marker


def verify_token_parts(root: Path) -> dict:
    root = Path(root)
    marker = json.loads((root / "DATA_READY.json").read_text())
    if marker.get("format") != FORMAT:
        raise ValueError("not a token-part dataset of this framework")
    seen = 0
    for p in marker["parts"]:
        data = (root / p["file"]).read_bytes()
        if len(data) != 4 * p["tokens"] or hashlib.sha256(data).hexdigest() != p["sha256"]:
            raise ValueError(f"part changed: {p['file']}")
        seen += p["tokens"]
    if seen != marker["tokens"]:
        raise ValueError("token count does not match the parts")
    return marker


def read_part(root: Path, index: int) -> np.ndarray:
    marker = json.loads((Path(root) / "DATA_READY.json").read_text())
    return np.fromfile(Path(root) / marker["parts"][index]["file"], dtype=np.int32)


_WS = re.compile(r"\s+")


def normalise_math_record(rec: dict, *, max_chars: int = 8000) -> dict | None:
    problem, answer = (rec.get("problem") or "").strip(), rec.get("answer")
    if not problem or answer is None or len(problem) > max_chars:
        return None
    canon = canonical_math_answer(str(answer))
    if canon is None:
        return None
    return {"problem": problem, "answer": canon, "key": hashlib.sha256(_WS.sub(" ", problem).lower().encode()).hexdigest(),
            "source": rec.get("source", "unknown")}


def filter_math_records(records: Iterable[dict], **kw) -> tuple[list[dict], dict]:
    kept, seen, stats = [], set(), {"read": 0, "invalid": 0, "duplicate": 0}
    for rec in records:
        stats["read"] += 1
        norm = normalise_math_record(rec, **kw)
        if norm is None:
            stats["invalid"] += 1
        elif norm["key"] in seen:
            stats["duplicate"] += 1
        else:
            seen.add(norm["key"])
            kept.append(norm)
    stats["kept"] = len(kept)
    return kept, stats


def split_by_group(group_id: str, seed: int, heldout_fraction: float) -> bool:
    """True when the group belongs to the held-out side."""
    h = int.from_bytes(hashlib.sha256(f"{seed}:{group_id}".encode()).digest()[:8], "big")
    return h / 2 ** 64 < heldout_fraction
