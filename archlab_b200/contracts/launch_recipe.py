"""Launch recipes for cluster jobs: a small allow-listed set of integer controls, resolved without running anything.

A launch recipe is ``{schema_version: 1, family, environment: {NGA_*: value}}``.  The resolver renders it to
``KEY=value`` bindings that a launcher exports; it never launches, and machine paths are not part of a recipe.  Rules:

* only the keys in ``KEYS`` may appear; every value except the model selector is an unsigned decimal integer that fits
  a signed 64-bit shell integer, printed WITHOUT leading zeros (shell arithmetic would read ``010`` as octal);
* a recipe names exactly one model family and one of that family's models; it must not carry the other family's
  selector; an environment variable that selects a different model than the recipe is a conflict, not an override;
* other environment variables override the recipe's defaults key by key (same validation);
* topology, batch and token-budget controls are required and positive; every pre-flight / probe control of the family
  must be set explicitly; an enabled pre-flight needs a positive number of steps.
The result also carries the family and the recipe's digest, which the run records.
(Reference: src/archlab/megatron/launch_config.py:17-89.)
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path
from typing import Mapping

from .recipe import read_recipe, recipe_sha256

KEYS = frozenset({"NGA_EXPECTED_NODES", "NGA_GPUS_PER_NODE", "NGA_SEQUENCE_LENGTH", "NGA_MICRO_BATCH_SIZE", "NGA_GLOBAL_BATCH_SIZE",
                  "NGA_TARGET_TRAIN_TOKENS", "NGA_CHECKPOINT_INTERVAL_TOKENS", "NGA_RUNTIME_PREFLIGHT", "NGA_PREFLIGHT_STEPS", "NGA_PROBE_STEPS",
                  "NGA_PROBE_SAVE_INTERVAL", "NGA_MODEL_SCALE", "NGA_FLASH_NEXT_MODEL_VARIANT"})
FAMILIES = {"dense-27b": ("NGA_MODEL_SCALE", {"quarter", "full"}),
            "flash-next": ("NGA_FLASH_NEXT_MODEL_VARIANT", {"full", "quarter-depth48-no-mtp", "1b-depth48-no-mtp", "w320-e32-depth48-no-mtp"})}
REQUIRED = ("NGA_EXPECTED_NODES", "NGA_GPUS_PER_NODE", "NGA_SEQUENCE_LENGTH", "NGA_MICRO_BATCH_SIZE", "NGA_GLOBAL_BATCH_SIZE", "NGA_TARGET_TRAIN_TOKENS",
            "NGA_CHECKPOINT_INTERVAL_TOKENS")
CONTROLS = {"dense-27b": ("NGA_PROBE_STEPS", "NGA_RUNTIME_PREFLIGHT", "NGA_PREFLIGHT_STEPS"), "flash-next": ("NGA_PROBE_STEPS", "NGA_PROBE_SAVE_INTERVAL")}


def resolve_launch_recipe(path, environment: Mapping[str, str]) -> dict[str, str]:
    recipe = read_recipe(path)
    if not isinstance(recipe, dict) or set(recipe) != {"schema_version", "family", "environment"}:
        raise ValueError("a launch recipe has exactly schema_version, family and environment")
    if type(recipe["schema_version"]) is not int or recipe["schema_version"] != 1 or recipe["family"] not in FAMILIES:
        raise ValueError("unsupported launch recipe schema or family")
    values, family = recipe["environment"], recipe["family"]
    if not isinstance(values, dict) or set(values) - KEYS:
        raise ValueError("the recipe contains unsupported environment keys")
    selector, models = FAMILIES[family]
    if values.get(selector) not in models:
        raise ValueError("the recipe must explicitly select a supported model")
    if any(FAMILIES[other][0] in values for other in FAMILIES if other != family):
        raise ValueError("the recipe mixes unrelated model families")
    if environment.get(selector) not in (None, "", values[selector]):
        raise ValueError(f"{selector} conflicts with the recipe; select the matching recipe explicitly")
    out = {}
    for key, default in values.items():
        value = environment.get(key) or str(default)
        if key != selector:
            if not value.isascii() or not value.isdecimal():
                raise ValueError(f"{key} must be an unsigned decimal integer")
            if int(value) > 2 ** 63 - 1:
                raise ValueError(f"{key} exceeds a signed 64-bit shell integer")
            value = str(int(value))
        out[key] = value
    if any(k not in out or int(out[k]) < 1 for k in REQUIRED):
        raise ValueError("the recipe needs positive topology, batch and token-budget controls")
    if any(k not in out for k in CONTROLS[family]):
        raise ValueError("the recipe must explicitly set every pre-flight / probe control")
    if out.get("NGA_RUNTIME_PREFLIGHT", "0") not in ("0", "1"):
        raise ValueError("runtime pre-flight must be 0 or 1")
    if out.get("NGA_RUNTIME_PREFLIGHT") == "1" and int(out.get("NGA_PREFLIGHT_STEPS", "0")) < 1:
        raise ValueError("an enabled pre-flight needs a positive number of steps")
    out["NGA_LAUNCH_FAMILY"] = family
    out["NGA_LAUNCH_RECIPE_SHA256"] = recipe_sha256(path)
    return out


def bindings(values: Mapping[str, str]) -> str:
    """``KEY=value`` lines; keys are allow-listed and values cannot contain a line feed, so no shell evaluation is needed."""
    return "\n".join(f"{k}={v}" for k, v in sorted(values.items()))


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--recipe", type=Path, required=True)
    ap.add_argument("--bindings", action="store_true")
    a = ap.parse_args(argv)
    values = resolve_launch_recipe(a.recipe, os.environ)
    print(bindings(values) if a.bindings else json.dumps(values, indent=2, sort_keys=True))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
