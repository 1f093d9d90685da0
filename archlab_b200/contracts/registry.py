"""Frozen campaign registry, per-backend capabilities and campaign variants.

* ``CAPABILITIES`` / ``require_backend_support``: which architecture variant has a validated adapter on
  which execution backend (src/archlab/capabilities.py:16-70).
* ``RunSpec`` + ``campaign_grid``: the frozen sizes x variants x seeds grid with the exact training
  command of every run (src/archlab/registry.py:36-168); ``verify_manifest`` checks a manifest is the
  complete Cartesian grid.
* ``VARIANTS``: per-variant model keyword arguments used by the campaigns
  (src/archlab/campaigns.py:28-467).
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any

SPEEDRUN_VARIANTS = ("attnres", "baseline", "dsa", "engram", "gated-attention", "glm-mla", "inkling-relative-attention",
                     "inkling-sconv-kv", "inkling-sconv-residual", "kda", "kimi-k3-kda-update", "mhc", "partial-rope-25",
                     "qwen-gdn", "situ-glu", "xielu")
# variants whose token mixer / residual runs on the mesh backend's fused tensor-parallel kernels
MESH_VARIANTS = ("baseline", "kda", "qwen-gdn", "dsa", "mhc", "simplicial")


@dataclass(frozen=True)
class ArchitectureCapability:
    variant: str
    speedrun: bool
    megatron: bool
    note: str = ""


CAPABILITIES = {v: ArchitectureCapability(v, True, v in MESH_VARIANTS,
                                          "fused peer-memory tensor-parallel adapter" if v in MESH_VARIANTS else
                                          "data-parallel speedrun only; needs a tensor-parallel adapter before scaling")
                for v in SPEEDRUN_VARIANTS}
CAPABILITIES["simplicial"] = ArchitectureCapability("simplicial", True, True, "2-simplicial attention layers (sm_100a kernels)")
CAPABILITIES["qwen2p5-1p5b-baseline"] = ArchitectureCapability("qwen2p5-1p5b-baseline", False, True,
                                                               "dense GQA backbone on the mesh backend")


def require_backend_support(variant: str, backend: str) -> None:
    cap = CAPABILITIES.get(variant)
    if cap is None:
        raise ValueError(f"unknown architecture variant: {variant}")
    if not getattr(cap, backend, False):
        raise ValueError(f"variant {variant!r} has no validated {backend} adapter; {cap.note}")


def capability_rows() -> list[dict[str, object]]:
    return [asdict(CAPABILITIES[k]) for k in sorted(CAPABILITIES)]


# ------------------------------------------------------------------------------------------------
# campaign variants: flags appended to the training command
# ------------------------------------------------------------------------------------------------
def arm_flags(model_kwargs: dict[str, Any]) -> tuple[str, ...]:
    """Model arguments of a campaign arm as trainer flags: ``--kda-pattern=KKKG``, tuples comma-separated, true
    booleans as bare flags (false ones are the trainer's defaults and are left out)."""
    out = []
    for key, value in model_kwargs.items():
        flag = "--" + key.replace("_", "-")
        if isinstance(value, bool):
            if value:
                out.append(flag)
        elif isinstance(value, (tuple, list)):
            out.append(f"{flag}={','.join(str(v) for v in value)}")
        else:
            out.append(f"{flag}={value}")
    return tuple(out)


def _variants() -> dict[str, tuple[str, ...]]:
    from .campaigns import TEN_M_VARIANTS

    return {v.name: arm_flags(v.model_kwargs()) for v in TEN_M_VARIANTS}


# the sixteen arms of the frozen campaign tables, as flags of ``archlab_b200.train.base_train``
VARIANTS: dict[str, tuple[str, ...]] = _variants()
SIZES = {"100m": dict(depth=12, aspect_ratio=64, head_dim=128), "300m": dict(depth=20, aspect_ratio=64, head_dim=128),
         "1b": dict(depth=28, aspect_ratio=80, head_dim=128)}
SEEDS = (0, 1, 2)
CAMPAIGN = "parameter-scale-100m-1b-v1"


@dataclass(frozen=True)
class RunSpec:
    run_id: str
    size_id: str
    variant_id: str
    seed: int
    parameter_count: int
    steps: int
    tokens: int
    depth: int
    aspect_ratio: int
    head_dim: int
    warmup_steps: int
    save_every: int
    variant_args: tuple[str, ...]

    @classmethod
    def from_dict(cls, payload: dict[str, Any]) -> "RunSpec":
        keys = ("run_id", "size_id", "variant_id", "seed", "parameter_count", "steps", "tokens", "depth", "aspect_ratio",
                "head_dim", "warmup_steps", "save_every")
        return cls(**{k: payload[k] for k in keys}, variant_args=tuple(payload["variant_args"]))

    def command(self, *, run_name: str = "dummy") -> list[str]:
        """The exact portable training command of this frozen run."""
        return ["python", "-m", "archlab_b200.train.base_train", f"--run={run_name}", f"--model-tag={self.run_id}",
                f"--seed={self.seed}", f"--depth={self.depth}", f"--aspect-ratio={self.aspect_ratio}",
                f"--head-dim={self.head_dim}", "--max-seq-len=2048", "--window-pattern=L", "--per-head-muon",
                "--device-batch-size=16", "--total-batch-size=393216", f"--num-iterations={self.steps}",
                f"--warmup-steps={self.warmup_steps}", "--warmdown-ratio=0.65", "--final-lr-frac=0.05",
                "--embedding-lr=0.3", "--unembedding-lr=0.008", "--matrix-lr=0.02", "--scalar-lr=0.5",
                "--weight-decay=0.28", "--eval-every=250", "--eval-tokens=3932160", f"--save-every={self.save_every}",
                "--finite-check-every=1", *self.variant_args]


def _dense_params(depth: int, aspect_ratio: int, vocab: int = 32768) -> int:
    d = depth * aspect_ratio
    return 12 * depth * d * d + 2 * vocab * d


def campaign_grid(tokens_per_param: float = 20.0, batch_tokens: int = 393216) -> list[RunSpec]:
    runs = []
    for size_id, geo in SIZES.items():
        n = _dense_params(geo["depth"], geo["aspect_ratio"])
        steps = max(1, round(tokens_per_param * n / batch_tokens))
        for variant, args in sorted(VARIANTS.items()):
            for seed in SEEDS:
                runs.append(RunSpec(f"{size_id}-{variant}-s{seed}", size_id, variant, seed, n, steps, steps * batch_tokens,
                                    geo["depth"], geo["aspect_ratio"], geo["head_dim"], max(10, steps // 50),
                                    max(1, steps // 4), args))
    return runs


def write_manifest(path: Path) -> dict:
    runs = campaign_grid()
    manifest = {"campaign": CAMPAIGN, "contract": {"sequence_length": 2048, "precision": "bfloat16"},
                "scope": {"total_runs": len(runs)}, "runs": [asdict(r) for r in runs]}
    Path(path).write_text(json.dumps(manifest, indent=1))
    return manifest


def load_runs(path: Path) -> list[RunSpec]:
    manifest = json.loads(Path(path).read_text())
    if manifest.get("campaign") != CAMPAIGN:
        raise ValueError(f"Unexpected campaign in {path}")
    return [RunSpec.from_dict(r) for r in manifest["runs"]]


def find_run(runs: list[RunSpec], size_id: str, variant_id: str, seed: int) -> RunSpec:
    hits = [r for r in runs if (r.size_id, r.variant_id, r.seed) == (size_id, variant_id, seed)]
    if len(hits) != 1:
        raise KeyError(f"Expected one run for size={size_id}, variant={variant_id}, seed={seed}; found {len(hits)}")
    return hits[0]


def verify_manifest(path: Path) -> dict[str, int]:
    manifest = json.loads(Path(path).read_text())
    runs = load_runs(path)
    keys = {(r.size_id, r.variant_id, r.seed) for r in runs}
    sizes, variants, seeds = {r.size_id for r in runs}, {r.variant_id for r in runs}, {r.seed for r in runs}
    if sizes != set(SIZES) or variants != set(VARIANTS) or seeds != set(SEEDS):
        raise ValueError("Manifest axes do not match the frozen campaign")
    expected = len(SIZES) * len(VARIANTS) * len(SEEDS)
    if len(runs) != expected or len(keys) != expected or len({r.run_id for r in runs}) != expected:
        raise ValueError(f"Manifest is not a complete Cartesian grid: {len(runs)} runs, {expected} expected")
    if manifest["contract"]["sequence_length"] != 2048 or manifest["contract"]["precision"] != "bfloat16":
        raise ValueError("Unexpected sequence length or precision")
    if manifest["scope"]["total_runs"] != expected:
        raise ValueError("Manifest total_runs disagrees with the frozen grid")
    if any(r.parameter_count <= 0 or r.steps <= 0 or r.tokens <= 0 or not r.variant_args for r in runs):
        raise ValueError("A run has invalid count or command metadata")
    return {"runs": len(runs), "sizes": len(sizes), "variants": len(variants), "seeds": len(seeds)}
