"""Layered, portable experiment specifications.

A specification is a YAML mapping, or one profile of a catalog (``FILE.yaml#PROFILE``), that may name parents
under ``extends``; parents are composed first, in order, and the file's own keys last (mappings merge key by key,
everything else is replaced).  Committed specifications carry no machine paths: every location is ``env:NAME``,
``package:relative/path`` or relative to the specification's own file.  The accepted surface is the one the
reference's loader accepts (src/archlab/spec.py:28-215): required keys ``schema_version, name, backend, variant,
seed``; ``paths`` / ``prompts`` portable; ``comparison`` and ``artifacts`` present together or not at all.

Structure: ``Reference`` classifies and resolves one location string; ``compose`` walks the ``extends`` graph with
an explicit work list; ``load_experiment`` runs a table of checks over the composed mapping.
"""
from __future__ import annotations

import copy
import os
import re
from collections.abc import Mapping
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from .recipe import read_recipe, split_recipe_reference
from .research import ArtifactPolicy, ComparisonContract, ContractError

PACKAGE_ROOT = Path(__file__).resolve().parent.parent
BACKENDS = ("speedrun", "megatron")
DEFAULT_PROMPTS = "package:prompts/smoke.yaml"


class SpecError(ValueError):
    """An experiment specification is incomplete, cyclic or not portable."""


def deep_merge(base: dict, update: Mapping) -> dict:
    """In-place layered merge: a mapping merges into a mapping, any other value replaces what was there."""
    pending = [(base, update)]
    while pending:
        into, new = pending.pop()
        for key, value in new.items():
            if isinstance(value, Mapping) and isinstance(into.get(key), dict):
                pending.append((into[key], value))
            else:
                into[key] = copy.deepcopy(value)
    return base


@dataclass(frozen=True)
class Reference:
    """One location string of a specification: ``env:NAME``, ``package:rel/path`` or a relative path."""
    scheme: str          # "env" | "package" | "relative"
    body: str

    _ENV = re.compile(r"[A-Z][A-Z0-9_]*")

    @classmethod
    def parse(cls, text: str, label: str) -> "Reference":
        for scheme in ("env", "package"):
            if text.startswith(scheme + ":"):
                ref = cls(scheme, text[len(scheme) + 1:])
                break
        else:
            ref = cls("relative", text)
        ref._check(text, label)
        return ref

    def _check(self, text: str, label: str) -> None:
        if self.scheme == "env" and not self._ENV.fullmatch(self.body):
            raise SpecError(f"{label}: {text!r} does not name an environment variable (UPPER_CASE)")
        if self.scheme == "package" and (Path(self.body).is_absolute() or ".." in Path(self.body).parts):
            raise SpecError(f"{label}: {text!r} must stay inside the package")
        if self.scheme == "relative" and Path(self.body).is_absolute():
            raise SpecError(f"{label}: absolute path {text!r} is not portable; write env:NAME or pass a CLI override")

    def resolve(self, anchor: Path, environ: Mapping[str, str]) -> str:
        if self.scheme == "env":
            value = environ.get(self.body)
            if not value:
                raise SpecError(f"required environment variable {self.body} is not set")
            return str(Path(value).expanduser().resolve())
        root = PACKAGE_ROOT if self.scheme == "package" else anchor
        return str((root / self.body).resolve())


def compose(reference) -> tuple[dict, list[Path]]:
    """Composed mapping of ``reference`` and the files it was built from (parents before children)."""
    def node_of(ref) -> tuple[Path, str | None]:
        file, profile = split_recipe_reference(ref)
        return file.resolve(), profile

    def read(node) -> tuple[dict, list]:
        file, profile = node
        try:
            value = read_recipe(f"{file}#{profile}" if profile else file)
        except ValueError as err:
            raise SpecError(str(err)) from err
        parents = value.pop("extends", [])
        parents = [parents] if isinstance(parents, str) else parents
        if not isinstance(parents, list) or not all(isinstance(p, str) for p in parents):
            raise SpecError(f"extends must be a string or list of strings: {file}")
        return value, [node_of(file.parent / p) for p in parents]

    show = lambda n: f"{n[0]}#{n[1]}" if n[1] else str(n[0])
    root = node_of(Path(str(reference)).expanduser())
    # depth-first with an explicit stack of (node, own mapping, parents still to visit, mapping built so far)
    merged_of: dict = {}
    sources: list[Path] = []
    own, parents = read(root)
    stack = [(root, own, list(parents), {})]
    while stack:
        node, own, todo, acc = stack[-1]
        if todo:
            parent = todo.pop(0)
            if any(parent == entry[0] for entry in stack):
                chain = " -> ".join(show(entry[0]) for entry in stack) + " -> " + show(parent)
                raise SpecError(f"cyclic experiment extends chain: {chain}")
            p_own, p_parents = read(parent)
            stack.append((parent, p_own, list(p_parents), {}))
            continue
        stack.pop()
        deep_merge(acc, own)
        sources.append(node[0])
        merged_of[node] = acc
        if stack:
            deep_merge(stack[-1][3], acc)
    return merged_of[root], sources


def _section(name: str):
    return property(lambda self: dict(self.config.get(name, {})))


@dataclass(frozen=True)
class ExperimentSpec:
    """A backend-neutral experiment contract plus the files it was composed from."""
    source: Path
    source_files: tuple[Path, ...]
    config: dict[str, Any]

    name = property(lambda self: str(self.config["name"]))
    backend = property(lambda self: str(self.config["backend"]))
    variant = property(lambda self: str(self.config["variant"]))
    seed = property(lambda self: int(self.config["seed"]))
    prompts = property(lambda self: str(self.config.get("prompts", DEFAULT_PROMPTS)))
    model, training, parallelism = _section("model"), _section("training"), _section("parallelism")

    def _contract(self, key: str, kind):
        raw = self.config.get(key)
        return None if raw is None else kind.from_mapping(raw)

    comparison = property(lambda self: self._contract("comparison", ComparisonContract))
    artifacts = property(lambda self: self._contract("artifacts", ArtifactPolicy))

    def resolve_reference(self, value: str, *, environ: Mapping[str, str] | None = None) -> str:
        return Reference.parse(value, "reference").resolve(self.source.parent, os.environ if environ is None else environ)

    def resolve_paths(self, overrides: Mapping[str, str] | None = None, *, environ: Mapping[str, str] | None = None) -> dict[str, str]:
        """Every configured path, resolved; an explicit override wins over the committed reference."""
        configured = self.config.get("paths", {})
        if not isinstance(configured, Mapping):
            raise SpecError("paths must be a mapping")
        overrides = dict(overrides or {})
        strangers = sorted(set(overrides) - set(configured))
        if strangers:
            raise SpecError(f"unknown path override(s): {', '.join(strangers)}")
        out = {}
        for key, committed in configured.items():
            out[key] = (str(Path(overrides[key]).expanduser().resolve()) if key in overrides
                        else self.resolve_reference(str(committed), environ=environ))
        return out


def _check_required(c):
    missing = sorted(k for k in ("schema_version", "name", "backend", "variant", "seed") if k not in c)
    return f"missing experiment key(s): {', '.join(missing)}" if missing else None


def _check_paths(c):
    paths = c.get("paths", {})
    if not isinstance(paths, Mapping):
        return "paths must be a mapping"
    for key, value in paths.items():
        if not isinstance(value, str):
            return f"path {key} must be a string"
        Reference.parse(value, f"paths.{key}")
    prompts = c.get("prompts", DEFAULT_PROMPTS)
    if not isinstance(prompts, str):
        return "prompts must be a portable string reference"
    Reference.parse(prompts, "prompts")
    return None


def _check_research(c):
    present = [k for k in ("comparison", "artifacts") if k in c]
    if not present:
        return None
    if len(present) != 2:
        return "new research specs must define both comparison and artifacts"
    for key in present:
        if not isinstance(c[key], Mapping):
            return f"{key} must be a mapping"
    try:
        ComparisonContract.from_mapping(c["comparison"])
        ArtifactPolicy.from_mapping(c["artifacts"])
    except ContractError as err:
        return str(err)
    return None


_CHECKS: tuple[Callable[[dict], str | None], ...] = (
    _check_required,
    lambda c: None if c["schema_version"] == 1 else f"unsupported schema_version: {c['schema_version']!r}",
    lambda c: None if c["backend"] in BACKENDS else f"unknown backend: {c['backend']!r}",
    lambda c: None if int(c["seed"]) >= 0 else "seed must be non-negative",
    _check_paths,
    _check_research,
)


def load_experiment(path) -> ExperimentSpec:
    """Load, compose and validate a portable experiment specification."""
    config, sources = compose(path)
    for check in _CHECKS:
        problem = check(config)
        if problem:
            raise SpecError(problem)
    file, _ = split_recipe_reference(Path(str(path)).expanduser())
    return ExperimentSpec(file.resolve(), tuple(sources), config)
