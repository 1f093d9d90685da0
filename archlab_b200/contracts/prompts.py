"""Versioned prompt sets shared by training-time sampling and evaluation entry points.

A prompt set is a YAML document ``{schema_version: 1, name: ..., prompts: [{id, text, tags?}, ...]}``: ids are unique,
texts are non-empty strings, tags are lists of strings.  Anything else is refused with the file named, so a sampling run
can never silently use a malformed or empty set (the reference's loader: src/archlab/prompts.py:12-46).  The packaged
default is ``prompt_sets/smoke.yaml``.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path

import yaml

SCHEMA_VERSION = 1
DEFAULT_SET = Path(__file__).resolve().parent.parent / "prompt_sets" / "smoke.yaml"


@dataclass(frozen=True)
class Prompt:
    id: str
    text: str
    tags: tuple[str, ...] = ()


def _refuse(path: Path, what: str):
    raise ValueError(f"{what}: {path}")


def load_prompt_set(path=None) -> tuple[Prompt, ...]:
    path = DEFAULT_SET if path is None else Path(path).expanduser().resolve()
    doc = yaml.safe_load(path.read_text(encoding="utf-8"))
    if not isinstance(doc, dict) or doc.get("schema_version") != SCHEMA_VERSION:
        _refuse(path, "unsupported prompt schema")
    rows = doc.get("prompts")
    if not isinstance(rows, list) or not rows:
        _refuse(path, "prompt set is empty")
    out: dict[str, Prompt] = {}
    for row in rows:
        if not isinstance(row, dict) or not isinstance(row.get("id"), str):
            _refuse(path, "invalid prompt row in")
        text, tags = row.get("text"), row.get("tags", [])
        if row["id"] in out or not isinstance(text, str) or not text:
            _refuse(path, f"invalid or duplicate prompt {row['id']!r} in")
        if not isinstance(tags, list) or not all(isinstance(t, str) for t in tags):
            _refuse(path, f"invalid tags for prompt {row['id']!r} in")
        out[row["id"]] = Prompt(row["id"], text, tuple(tags))
    return tuple(out.values())


def prompt_texts(path=None, *, tag: str | None = None) -> list[str]:
    return [p.text for p in load_prompt_set(path) if tag is None or tag in p.tags]
