"""``archlab {resolve|qualify|train} RECIPE --overlay O --output DIR [key=value ...]``.

The one public console entry (the reference exposes the same function under two script names,
``archlab`` and ``next-gen-arch``: pyproject.toml:42-44, src/archlab/training/cli.py:15-41).
``resolve`` writes ``resolved.yaml`` + ``experiment.json``; ``qualify`` adds ``qualification.json``;
``train`` launches only when qualification passed.
"""
from __future__ import annotations

import argparse
from dataclasses import asdict
from pathlib import Path

import yaml

from .contracts.experiment import compose_trainer, read_experiment
from .contracts.substrate import atomic_write_json

ACTIONS = ("resolve", "qualify", "train")


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="archlab", description="Resolve, qualify or launch one experiment recipe")
    p.add_argument("action", choices=ACTIONS)
    p.add_argument("recipe", type=Path)
    p.add_argument("--output", type=Path, required=True)
    p.add_argument("--overlay", type=Path, action="append", default=[])
    p.add_argument("--config-root", type=Path, default=None, help="directory holding the trainer configuration trees (default: packaged)")
    p.add_argument("--skip-gates", action="store_true", help="qualify: readiness checks only")
    p.add_argument("overrides", nargs="*")
    return p


def resolve(args):
    """Writes the resolved trainer configuration and the typed experiment; returns both."""
    experiment = read_experiment(args.recipe, args.overrides, overlays=args.overlay)
    config = compose_trainer(experiment, args.config_root)
    args.output.mkdir(parents=True, exist_ok=True)
    (args.output / "resolved.yaml").write_text(yaml.safe_dump(config, sort_keys=False))
    atomic_write_json(args.output / "experiment.json", asdict(experiment))
    return experiment, config


def main(argv=None) -> int:
    args = build_parser().parse_intermixed_args(argv)
    experiment, config = resolve(args)
    if args.action == "resolve":
        return 0
    from .train.qualification import qualify

    verdict = qualify(experiment, config, args.output, run_gates=not args.skip_gates)
    if not verdict["passed"]:
        print("Qualification blocked; see", args.output / "qualification.json")
        return 1
    if args.action == "train":
        from .train.runtime import run

        run(experiment, config, args.output)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
