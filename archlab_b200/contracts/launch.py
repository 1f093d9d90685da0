"""Launch plans: an inspectable argv + environment + provenance bundle
(src/archlab/launch.py:11-57).  ``env:NAME`` tokens render as ``"${NAME}"`` so a committed plan
stays free of machine paths."""
from __future__ import annotations

import json
import re
import shlex
from collections.abc import Mapping
from dataclasses import dataclass, field
from typing import Any

_ENV_TOKEN = re.compile(r"^env:([A-Z][A-Z0-9_]*)$")


def shell_token(token: str) -> str:
    m = _ENV_TOKEN.fullmatch(token)
    return f'"${{{m.group(1)}}}"' if m else shlex.quote(token)


@dataclass(frozen=True)
class LaunchPlan:
    backend: str
    argv: tuple[str, ...]
    env: Mapping[str, str] = field(default_factory=dict)
    metadata: Mapping[str, Any] = field(default_factory=dict)

    def shell(self) -> str:
        prefix = [f"{k}={shlex.quote(v)}" for k, v in sorted(self.env.items())]
        return " ".join([*prefix, *(shell_token(t) for t in self.argv)])

    def as_dict(self) -> dict[str, Any]:
        return {"backend": self.backend, "argv": list(self.argv), "env": dict(self.env),
                "metadata": dict(self.metadata)}

    def json(self) -> str:
        return json.dumps(self.as_dict(), indent=2, sort_keys=True) + "\n"


def get_backend(name: str):
    """``speedrun`` (single-mesh data parallel) or ``megatron`` (TP/PP/CP/EP mesh) launch renderers."""
    from ..train import backends

    if name == "speedrun":
        return backends.SpeedrunBackend()
    if name == "megatron":
        return backends.MeshBackend()
    raise ValueError(f"unknown backend: {name}")
