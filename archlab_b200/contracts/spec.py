"""Layered, portable experiment specifications (src/archlab/spec.py:28-215).

A spec is YAML with optional ``extends: [FILE.yaml#PROFILE, ...]`` parents (merged depth-first,
cycles rejected), required keys ``schema_version, name, backend, variant, seed`` and portable path
references only: ``env:NAME``, ``package:relative/path`` or a path relative to the spec file.
"""
from __future__ import annotations

import copy
import os
import re
from collections.abc import Mapping
from dataclasses import dataclass
from pathlib import Path
from typing import Any

from .recipe import read_recipe, split_recipe_reference
from .research import ArtifactPolicy, ComparisonContract, ContractError

PACKAGE_ROOT = Path(__file__).resolve().parent.parent
_ENV_NAME = re.compile(r"^[A-Z][A-Z0-9_]*$")
REQUIRED = ("schema_version", "name", "backend", "variant", "seed")


class SpecError(ValueError):
    pass


def deep_merge(base: dict, update: Mapping) -> dict:
    """Mappings merge recursively; scalars and sequences are replaced."""
    for k, v in update.items():
        if isinstance(v, Mapping) and isinstance(base.get(k), dict):
            deep_merge(base[k], v)
        else:
            base[k] = copy.deepcopy(v)
    return base


def _load_layered(reference: Path, stack: tuple = ()) -> tuple[dict, list[Path]]:
    file, profile = split_recipe_reference(reference)
    key = (file.resolve(), profile)
    if key in stack:
        raise SpecError("cyclic experiment extends chain: " + " -> ".join(f"{p}#{q}" if q else str(p)
                                                                          for p, q in (*stack, key)))
    try:
        value = read_recipe(f"{file.resolve()}#{profile}" if profile else file.resolve())
    except ValueError as e:
        raise SpecError(str(e)) from e
    extends = value.pop("extends", [])
    if isinstance(extends, str):
        extends = [extends]
    if not isinstance(extends, list) or not all(isinstance(x, str) for x in extends):
        raise SpecError(f"extends must be a string or list of strings: {file}")
    merged: dict = {}
    sources: list[Path] = []
    for ref in extends:
        pv, ps = _load_layered(file.resolve().parent / ref, (*stack, key))
        deep_merge(merged, pv)
        sources.extend(ps)
    deep_merge(merged, value)
    sources.append(file.resolve())
    return merged, sources


def validate_portable_reference(value: str, label: str) -> None:
    if value.startswith("env:"):
        if not _ENV_NAME.fullmatch(value[4:]):
            raise SpecError(f"invalid environment reference for {label}: {value!r}")
        return
    if value.startswith("package:"):
        rel = Path(value[8:])
        if rel.is_absolute() or ".." in rel.parts:
            raise SpecError(f"invalid package reference for {label}: {value!r}")
        return
    if Path(value).is_absolute():
        raise SpecError(f"committed path {label} must be portable, got absolute path {value!r}; "
                        "use env:NAME or a CLI override")


@dataclass(frozen=True)
class ExperimentSpec:
    source: Path
    source_files: tuple[Path, ...]
    config: dict[str, Any]

    name = property(lambda s: str(s.config["name"]))
    backend = property(lambda s: str(s.config["backend"]))
    variant = property(lambda s: str(s.config["variant"]))
    seed = property(lambda s: int(s.config["seed"]))
    prompts = property(lambda s: str(s.config.get("prompts", "package:prompts/smoke.yaml")))
    model = property(lambda s: dict(s.config.get("model", {})))
    training = property(lambda s: dict(s.config.get("training", {})))
    parallelism = property(lambda s: dict(s.config.get("parallelism", {})))

    @property
    def comparison(self) -> ComparisonContract | None:
        v = self.config.get("comparison")
        return None if v is None else ComparisonContract.from_mapping(v)

    @property
    def artifacts(self) -> ArtifactPolicy | None:
        v = self.config.get("artifacts")
        return None if v is None else ArtifactPolicy.from_mapping(v)

    def resolve_reference(self, value: str, *, environ: Mapping[str, str] | None = None) -> str:
        environ = os.environ if environ is None else environ
        if value.startswith("env:"):
            got = environ.get(value[4:])
            if not got:
                raise SpecError(f"required environment variable {value[4:]} is not set")
            return str(Path(got).expanduser().resolve())
        if value.startswith("package:"):
            return str((PACKAGE_ROOT / value[8:]).resolve())
        return str((self.source.parent / value).resolve())

    def resolve_paths(self, overrides: Mapping[str, str] | None = None, *,
                      environ: Mapping[str, str] | None = None) -> dict[str, str]:
        overrides = dict(overrides or {})
        configured = self.config.get("paths", {})
        if not isinstance(configured, Mapping):
            raise SpecError("paths must be a mapping")
        unknown = set(overrides) - set(configured)
        if unknown:
            raise SpecError(f"unknown path override(s): {', '.join(sorted(unknown))}")
        return {k: str(Path(overrides[k]).expanduser().resolve()) if k in overrides
                else self.resolve_reference(str(v), environ=environ) for k, v in configured.items()}


def load_experiment(path: str | Path) -> ExperimentSpec:
    ref = Path(str(path)).expanduser()
    file, _ = split_recipe_reference(ref)
    config, sources = _load_layered(ref)
    missing = [k for k in REQUIRED if k not in config]
    if missing:
        raise SpecError(f"missing experiment key(s): {', '.join(sorted(missing))}")
    if config["schema_version"] != 1:
        raise SpecError(f"unsupported schema_version: {config['schema_version']!r}")
    if config["backend"] not in {"speedrun", "megatron"}:
        raise SpecError(f"unknown backend: {config['backend']!r}")
    if int(config["seed"]) < 0:
        raise SpecError("seed must be non-negative")
    paths = config.get("paths", {})
    if not isinstance(paths, Mapping):
        raise SpecError("paths must be a mapping")
    for k, v in paths.items():
        if not isinstance(v, str):
            raise SpecError(f"path {k} must be a string")
        validate_portable_reference(v, f"paths.{k}")
    prompts = config.get("prompts", "package:prompts/smoke.yaml")
    if not isinstance(prompts, str):
        raise SpecError("prompts must be a portable string reference")
    validate_portable_reference(prompts, "prompts")
    research = {k for k in ("comparison", "artifacts") if k in config}
    if research and research != {"comparison", "artifacts"}:
        raise SpecError("new research specs must define both comparison and artifacts")
    if research:
        for k in research:
            if not isinstance(config[k], Mapping):
                raise SpecError(f"{k} must be a mapping")
        try:
            ComparisonContract.from_mapping(config["comparison"])
            ArtifactPolicy.from_mapping(config["artifacts"])
        except ContractError as e:
            raise SpecError(str(e)) from e
    return ExperimentSpec(file.resolve(), tuple(sources), config)
