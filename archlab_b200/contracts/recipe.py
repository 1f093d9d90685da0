"""Recipe files: a standalone YAML mapping, or a catalog ``{profiles: {NAME: {...}}}`` addressed as
``FILE.yaml#PROFILE``.  A profile is never inferred from a path or an output name: a catalog without ``#PROFILE`` is an
error, and so is a profile the catalog does not define (src/archlab/recipe.py:14-46)."""
from __future__ import annotations

import copy
import hashlib
import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any

import yaml


@dataclass(frozen=True)
class RecipeRef:
    """``path`` plus the optional profile named after ``#``."""
    path: Path
    profile: str | None

    @classmethod
    def parse(cls, reference) -> "RecipeRef":
        text = str(reference)
        file, has_marker, name = text.partition("#")
        if file == "" or (has_marker and name == ""):
            raise ValueError("recipe reference needs a path and a nonempty profile after #")
        return cls(Path(file), name if has_marker else None)

    def document(self) -> dict:
        loaded = yaml.safe_load(self.path.read_text(encoding="utf-8"))
        if not isinstance(loaded, dict):
            raise ValueError(f"recipe must be a mapping: {self.path}")
        return loaded

    def select(self) -> dict[str, Any]:
        document = self.document()
        if self.profile is None:
            if "profiles" in document:
                raise ValueError(f"catalog requires an explicit #PROFILE: {self.path}")
            return copy.deepcopy(document)
        catalog = document.get("profiles")
        if not isinstance(catalog, dict) or self.profile not in catalog:
            raise ValueError(f"unknown recipe profile {self.profile!r} in {self.path}")
        chosen = catalog[self.profile]
        if not isinstance(chosen, dict):
            raise ValueError(f"recipe profile must be a mapping: {self.path}#{self.profile}")
        return copy.deepcopy(chosen)

    def sha256(self) -> str:
        """Standalone recipes hash as the file's bytes (what earlier receipts recorded); a catalog profile hashes as the
        canonical JSON of the selected mapping, so editing ANOTHER profile of the catalog does not change it."""
        if self.profile is None:
            return hashlib.sha256(self.path.read_bytes()).hexdigest()
        canonical = json.dumps(self.select(), sort_keys=True, separators=(",", ":"))
        return hashlib.sha256(canonical.encode()).hexdigest()


def split_recipe_reference(reference: str | Path) -> tuple[Path, str | None]:
    ref = RecipeRef.parse(reference)
    return ref.path, ref.profile


def read_recipe(reference: str | Path) -> dict[str, Any]:
    return RecipeRef.parse(reference).select()


def recipe_sha256(reference: str | Path) -> str:
    return RecipeRef.parse(reference).sha256()
