"""Recipe files: a standalone YAML mapping, or a catalog ``{profiles: {NAME: {...}}}`` addressed as
``FILE.yaml#PROFILE``.  A profile is never inferred (src/archlab/recipe.py:14-46)."""
from __future__ import annotations

import copy
import hashlib
import json
from pathlib import Path
from typing import Any

import yaml


def split_recipe_reference(reference: str | Path) -> tuple[Path, str | None]:
    path, marker, profile = str(reference).partition("#")
    if not path or (marker and not profile):
        raise ValueError("recipe reference needs a path and a nonempty profile after #")
    return Path(path), (profile if marker else None)


def read_recipe(reference: str | Path) -> dict[str, Any]:
    path, profile = split_recipe_reference(reference)
    value = yaml.safe_load(path.read_text(encoding="utf-8"))
    if not isinstance(value, dict):
        raise ValueError(f"recipe must be a mapping: {reference}")
    if profile is None:
        if "profiles" in value:
            raise ValueError(f"catalog requires an explicit #PROFILE: {path}")
        return copy.deepcopy(value)
    profiles = value.get("profiles")
    if not isinstance(profiles, dict) or profile not in profiles:
        raise ValueError(f"unknown recipe profile {profile!r} in {path}")
    if not isinstance(profiles[profile], dict):
        raise ValueError(f"recipe profile must be a mapping: {reference}")
    return copy.deepcopy(profiles[profile])


def recipe_sha256(reference: str | Path) -> str:
    """Raw file hash for standalone recipes; canonical-JSON hash of the selected profile otherwise."""
    path, profile = split_recipe_reference(reference)
    if profile is None:
        return hashlib.sha256(path.read_bytes()).hexdigest()
    payload = json.dumps(read_recipe(reference), sort_keys=True, separators=(",", ":")).encode()
    return hashlib.sha256(payload).hexdigest()
