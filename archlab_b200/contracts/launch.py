"""Launch plans: what a backend would run, kept inspectable -- the argument vector, the environment it adds and the
provenance that explains both (src/archlab/launch.py:11-57).

Arguments of the form ``env:NAME`` stand for a value the launching machine supplies; they render as ``"${NAME}"`` in
the shell form, so a committed plan never contains a machine path, and every other token is shell-quoted.
"""
from __future__ import annotations

import json
import re
import shlex
from collections.abc import Mapping
from dataclasses import dataclass, field
from typing import Any

ENV_REFERENCE = re.compile(r"env:([A-Z][A-Z0-9_]*)")
BACKENDS = {"speedrun": "SpeedrunBackend", "megatron": "MeshBackend"}      # single-mesh data parallel / TP-PP-CP-EP mesh


def shell_token(token: str) -> str:
    reference = ENV_REFERENCE.fullmatch(token)
    if reference is None:
        return shlex.quote(token)
    return '"${' + reference.group(1) + '}"'


@dataclass(frozen=True)
class LaunchPlan:
    backend: str
    argv: tuple[str, ...]
    env: Mapping[str, str] = field(default_factory=dict)
    metadata: Mapping[str, Any] = field(default_factory=dict)

    def environment_assignments(self) -> list[str]:
        return [name + "=" + shlex.quote(self.env[name]) for name in sorted(self.env)]

    def shell(self) -> str:
        """One line: sorted ``NAME=value`` assignments, then the command."""
        return " ".join(self.environment_assignments() + [shell_token(t) for t in self.argv])

    def as_dict(self) -> dict[str, Any]:
        return dict(backend=self.backend, argv=[*self.argv], env={**self.env}, metadata={**self.metadata})

    def json(self) -> str:
        return json.dumps(self.as_dict(), sort_keys=True, indent=2) + "\n"


def get_backend(name: str):
    if name not in BACKENDS:
        raise ValueError(f"unknown backend: {name}")
    from ..train import backends

    return getattr(backends, BACKENDS[name])()
