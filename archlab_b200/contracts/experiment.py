"""Typed experiment contract, overlay / override merge and fail-closed science validators.

Mirrors the behaviour of the reference's ``archlab.training.config`` (``Experiment`` dataclass
:18-50, ``read_experiment`` :53-106, composition :109-146, ``validate_science`` :149-349,
``fingerprint`` :352-353) without OmegaConf / Hydra: recipes and overlays are plain YAML merged
in order onto the dataclass defaults, trailing ``key=value`` overrides update typed fields, and
``settings.<dotted.path>=value`` writes a literal path of the composed trainer configuration tree
(which is struct-checked: an unknown path is an error, never a silent new key).
``${oc.env:NAME[,default]}`` interpolations are resolved when the tree is composed.
"""
from __future__ import annotations

import copy
import dataclasses
import hashlib
import json
import math
import os
import re
from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Any

import yaml

from .performance import ThroughputContract

MISSING = "???"
FAMILIES = {"limite", "muse_glimmer", "qwen3_5", "speedrun"}
VARIANTS = {"normal", "simplicial", "linsimp", "triadic"}
INTERVENTIONS = {"insert_attention", "replace_attention", "none"}
ENGINES = {"megatron", "dp"}
ATTENTION = {"native", "tilelang", "te"}
EXECUTION = {"sync", "colocate_async"}
CONFIG_ROOT = Path(__file__).resolve().parent.parent / "config_tree"


@dataclass
class AgenticPilot:
    max_turn_tokens: int = 8192
    step_limit: int = 500
    minimum_prompt_groups: int = 2
    minimum_completed_verifiers: int = 8
    minimum_tool_calls: int = 1
    minimum_observation_tokens: int = 1
    minimum_reward_contrast_groups: int = 1
    maximum_truncated_trajectories: int = 0


@dataclass
class Experiment:
    name: str = MISSING
    family: str = "limite"
    variant: str = "normal"
    intervention: str = "insert_attention"
    engine: str = "megatron"
    attention: str = "tilelang"
    execution: str = "colocate_async"
    native_context: int = 131072
    parent_checkpoint: str = MISSING
    parent_stage: str = "adapter_sft"
    parent_tokens: int | None = 2_000_158_720
    publisher_manifest: str | None = None
    data_manifest: str = MISSING
    resume_checkpoint: str | None = None
    maximum_policy_lag: int = 1
    pilot: AgenticPilot | None = None
    throughput: ThroughputContract = field(default_factory=ThroughputContract)
    settings: dict[str, Any] = field(default_factory=dict)


# ------------------------------------------------------------------------------------------------
# merge
# ------------------------------------------------------------------------------------------------
def parse_scalar(raw: str) -> Any:
    """YAML scalar / flow syntax, the same value grammar a dotlist override uses."""
    try:
        return yaml.safe_load(raw)
    except yaml.YAMLError:
        return raw


def _coerce(value: Any, typ: Any, label: str) -> Any:
    if value is None:
        return None
    origin = getattr(typ, "__origin__", None)
    if typ in (int, "int") or str(typ) in ("int | None", "int"):
        if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value:
            raise ValueError(f"{label} must be an integer")
        return int(value)
    if typ in (str,) or str(typ) in ("str | None", "str"):
        return str(value)
    if origin is dict or typ is dict:
        if not isinstance(value, dict):
            raise ValueError(f"{label} must be a mapping")
        return dict(value)
    return value


def _build_dataclass(cls, data: dict, label: str):
    known = {f.name: f for f in fields(cls)}
    unknown = set(data) - set(known)
    if unknown:
        raise ValueError(f"unknown key(s) in {label}: {', '.join(sorted(unknown))}")
    kwargs = {}
    for name, f in known.items():
        if name not in data:
            continue
        v = data[name]
        if name == "pilot":
            kwargs[name] = None if v is None else _build_dataclass(AgenticPilot, dict(v), "pilot")
        elif name == "throughput":
            kwargs[name] = _build_dataclass(ThroughputContract, dict(v or {}), "throughput")
        else:
            kwargs[name] = _coerce(v, f.type, f"{label}.{name}" if label else name)
    return cls(**kwargs)


def _deep_merge(base: dict, update: dict) -> dict:
    for k, v in update.items():
        if isinstance(v, dict) and isinstance(base.get(k), dict):
            _deep_merge(base[k], v)
        else:
            base[k] = copy.deepcopy(v)
    return base


def _set_dotted(tree: dict, dotted: str, value: Any, *, struct: bool, label: str = "") -> None:
    node = tree
    parts = dotted.split(".")
    for i, part in enumerate(parts[:-1]):
        if not isinstance(node, dict) or part not in node:
            if struct:
                raise KeyError(f"unknown configuration path {label}{'.'.join(parts[:i + 1])}")
            node = node.setdefault(part, {})
        else:
            node = node[part]
    if struct and (not isinstance(node, dict) or parts[-1] not in node):
        raise KeyError(f"unknown configuration path {label}{dotted}")
    node[parts[-1]] = value


def read_experiment(path: str | Path, overrides: list[str] | tuple[str, ...] = (), *,
                    overlays: list[Path] | tuple[Path, ...] = ()) -> Experiment:
    data: dict = {}
    for src in (path, *overlays):
        loaded = yaml.safe_load(Path(src).read_text(encoding="utf-8")) or {}
        if not isinstance(loaded, dict):
            raise ValueError(f"recipe must be a mapping: {src}")
        settings = loaded.pop("settings", None)
        _deep_merge(data, loaded)
        if settings:
            # settings keys are literal dotted upstream paths; later files replace whole values
            data.setdefault("settings", {}).update(settings)
    for ov in overrides:
        key, sep, raw = ov.partition("=")
        if not sep or not key:
            raise ValueError("overrides must use key=value")
        value = parse_scalar(raw)
        if key.startswith("settings."):
            data.setdefault("settings", {})[key[len("settings."):]] = value
        else:
            _set_dotted(data, key, value, struct=False)
    # experiment fields interpolate environment variables like the trainer tree does; a variable that is not set
    # (and has no default) stays as written, so a recipe can be read and checked without its deployment environment
    for key in list(data):
        if key != "settings":
            data[key] = _resolve_env(data[key], os.environ, strict=False)
    exp = _build_dataclass(Experiment, data, "")
    for req in ("name", "parent_checkpoint", "data_manifest"):
        if getattr(exp, req) == MISSING:
            raise ValueError(f"missing mandatory value: {req}")
    validate_experiment(exp)
    return exp


def validate_experiment(e: Experiment) -> None:
    """Cross-field rules of the typed contract (reference :68-105)."""
    e.throughput.validate()
    if e.family not in FAMILIES:
        raise ValueError("unknown model family")
    if e.family == "limite" and e.engine != "megatron":
        raise ValueError("the primary execution engine is megatron")
    if e.engine not in ENGINES:
        raise ValueError("engine must be megatron or dp")
    if e.attention not in ATTENTION:
        raise ValueError("attention must be native, tilelang or te")
    if e.execution not in EXECUTION:
        raise ValueError("execution must be sync or colocate_async")
    if e.variant not in VARIANTS:
        raise ValueError("unknown architecture variant")
    if e.intervention not in INTERVENTIONS:
        raise ValueError("unknown architecture intervention")
    if e.native_context <= 0:
        raise ValueError("native_context must be positive")
    if e.maximum_policy_lag < 0:
        raise ValueError("maximum_policy_lag must be nonnegative")
    if e.family == "speedrun":
        return   # pre-training runs on this framework's own trainer; no RL lineage rules apply
    if e.family != "qwen3_5" and e.maximum_policy_lag != 1:
        raise ValueError("the existing Limite and Muse pilots permit at most one policy version of lag")
    if e.resume_checkpoint and e.family != "qwen3_5":
        raise ValueError("the existing Limite and Muse pilots require fresh RL")
    if e.family in {"muse_glimmer", "qwen3_5"}:
        if (e.engine != "dp" or e.variant != "normal" or e.attention != "native" or e.intervention != "none"
                or e.parent_stage != "published_checkpoint" or e.parent_tokens is not None
                or not e.publisher_manifest):
            raise ValueError("native control requires DP, unchanged publisher weights and an asset manifest")
    elif e.intervention == "none":
        raise ValueError("Limite requires its explicit attention intervention")
    elif e.parent_stage == "package_sft":
        if (e.intervention != "replace_attention" or e.variant != "simplicial" or e.attention != "tilelang"
                or e.parent_tokens is not None):
            raise ValueError("package SFT replacement uses simplicial TileLang and receipt-derived token budgets")
    elif e.parent_stage not in {"adapter_sft", "full_sft"} or e.parent_tokens is None or e.parent_tokens <= 0:
        raise ValueError("this fresh RL pilot requires an explicit SFT token endpoint")
    if e.intervention == "replace_attention" and e.parent_stage != "package_sft":
        raise ValueError("attention replacement RL requires a trained package SFT endpoint")


def experiment_dict(e: Experiment) -> dict:
    return dataclasses.asdict(e)


def fingerprint(config: Any) -> str:
    """sha256 of the canonical JSON of a resolved configuration."""
    return hashlib.sha256(json.dumps(config, sort_keys=True, default=str).encode()).hexdigest()


# ------------------------------------------------------------------------------------------------
# composition of the trainer configuration tree
# ------------------------------------------------------------------------------------------------
class Tree(dict):
    """dict with attribute access (read-only convenience for the validators)."""

    def __getattr__(self, k):
        try:
            v = self[k]
        except KeyError as e:
            raise AttributeError(k) from e
        return Tree(v) if isinstance(v, dict) and not isinstance(v, Tree) else v


_INTERP = re.compile(r"\$\{oc\.env:([A-Za-z_][A-Za-z0-9_]*)(?:,([^}]*))?\}")


def _resolve_env(value: Any, environ, strict: bool = True) -> Any:
    if isinstance(value, dict):
        return {k: _resolve_env(v, environ, strict) for k, v in value.items()}
    if isinstance(value, list):
        return [_resolve_env(v, environ, strict) for v in value]
    if isinstance(value, str):
        whole = _INTERP.fullmatch(value)

        def sub(m):
            got = environ.get(m.group(1), m.group(2))
            if got is None:
                if not strict:
                    return m.group(0)
                raise ValueError(f"environment variable {m.group(1)} is not set and has no default")
            return str(got)

        if whole:
            return parse_scalar(sub(whole))
        return _INTERP.sub(sub, value)
    return value


def _find_missing(tree: Any, prefix: str = "") -> list[str]:
    out = []
    if isinstance(tree, dict):
        for k, v in tree.items():
            out += _find_missing(v, f"{prefix}{k}.")
    elif tree == MISSING:
        out.append(prefix[:-1])
    return out


def compose_trainer(experiment: Experiment, config_root: Path | None = None, *, environ=None,
                    validate: bool = True) -> dict:
    """Build the resolved trainer configuration: base tree for the engine, then every
    ``settings`` entry written to its literal dotted path (struct-checked), then the experiment-
    derived fields, environment interpolation and the science validators."""
    root = Path(config_root) if config_root is not None else CONFIG_ROOT
    name = "ppo_trainer.yaml" if experiment.engine == "dp" else "train.yaml"
    tree = yaml.safe_load((root / name).read_text(encoding="utf-8"))
    tree["model_engine"] = experiment.engine
    for key, value in experiment.settings.items():
        try:
            _set_dotted(tree, key, copy.deepcopy(value), struct=True, label="settings.")
        except KeyError as e:
            raise ValueError(str(e.args[0])) from e
    tree["trainer"]["experiment_name"] = experiment.name
    tree["trainer"]["use_v1"] = True
    tree["trainer"]["v1"]["trainer_mode"] = experiment.execution
    if not tree["reward"]["reward_model"]["enable"]:
        tree["reward"]["reward_model"]["rollout"]["name"] = None
    tree = _resolve_env(tree, os.environ if environ is None else environ)
    if validate and experiment.family != "speedrun":
        validate_science(experiment, tree)
    missing = _find_missing(tree)
    if missing:
        raise ValueError(f"missing mandatory value(s): {', '.join(missing)}")
    return tree


def validate_science(experiment: Experiment, config: dict) -> None:
    """Fail-closed invariants of the agentic RL pilots; the rules are the table in ``science_rules`` and the raised
    ``ValueError`` carries the violated rule's message (and the offending path as ``violated_path``)."""
    from . import science_rules

    science_rules.validate(experiment, config)
