"""Proof that a change to sealed source is formatting-only: the AST (without docstring-free
normalisation of layout) must hash identically (src/archlab/source_compatibility.py:14-45)."""
from __future__ import annotations

import ast
import hashlib
from pathlib import Path


def ast_sha256(source: str) -> str:
    return hashlib.sha256(ast.dump(ast.parse(source), include_attributes=False).encode()).hexdigest()


def formatting_only_change(before: str, after: str) -> bool:
    return ast_sha256(before) == ast_sha256(after)


def prove_compatible(sealed: dict[str, str], root) -> dict[str, str]:
    """``sealed`` maps relative path -> AST hash recorded when the source was sealed; raises on any file
    whose syntax tree changed."""
    out = {}
    for rel, want in sorted(sealed.items()):
        got = ast_sha256((Path(root) / rel).read_text(encoding="utf-8"))
        if got != want:
            raise ValueError(f"sealed source changed beyond formatting: {rel}")
        out[rel] = got
    return out
