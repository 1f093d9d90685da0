"""``archlab train``: executes a qualified experiment on this machine's GPUs.

The launch itself is a ``LaunchPlan`` (``train/backends.py``) rendered from the experiment's engine and
settings, written next to the resolved configuration, then started as a child ``torch.distributed.run``
process group.  Private tracking settings are handed to workers through the environment only
(never written into plans or receipts), following src/archlab/training/runtime.py:14-80.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

from ..contracts.substrate import atomic_write_json
from .backends import MeshBackend, SpeedrunBackend, Topology


def _setting(experiment, key: str, default):
    return (experiment.settings or {}).get(key, default)


def plan_for(experiment, config: dict, output: Path, *, gpus: int | None = None):
    """Experiment -> LaunchPlan.  ``engine == 'speedrun'`` is the data-parallel speedrun; anything else
    is a model-parallel mesh run."""
    import torch

    n = gpus or max(torch.cuda.device_count(), 1)
    topo = Topology(nodes=int(_setting(experiment, "nodes", 1)), gpus_per_node=n,
                    master_port=int(_setting(experiment, "master_port", 29500)))
    run_dir = str(Path(output) / "run")
    if experiment.engine == "speedrun":
        return SpeedrunBackend().render(
            depth=int(_setting(experiment, "depth", 20)), device_batch_size=int(_setting(experiment, "device_batch_size", 16)),
            total_batch_size=int(_setting(experiment, "total_batch_size", 524288 // 8 * n)),
            max_seq_len=int(_setting(experiment, "max_seq_len", 2048)),
            num_iterations=int(_setting(experiment, "num_iterations", -1)), run_dir=run_dir, topology=topo)
    return MeshBackend().render(
        model=str(_setting(experiment, "model", experiment.family)), tp=int(_setting(experiment, "tp", 1)),
        pp=int(_setting(experiment, "pp", 1)), cp=int(_setting(experiment, "cp", 1)), ep=int(_setting(experiment, "ep", 1)),
        micro_batch=int(_setting(experiment, "micro_batch", 1)), global_batch=int(_setting(experiment, "global_batch", 8 * n)),
        seq_len=int(_setting(experiment, "seq_len", 8192)), precision=str(_setting(experiment, "precision", "bf16")),
        run_dir=run_dir, topology=topo)


def worker_environment(base: dict | None = None) -> dict:
    """Environment of the launched ranks: the caller's, plus tracking settings loaded from the private
    file named by ``ARCHLAB_MLFLOW_CONFIG`` (the values travel in memory only)."""
    env = dict(os.environ if base is None else base)
    if path := env.get("ARCHLAB_MLFLOW_CONFIG"):
        tracking = json.loads(Path(path).read_text())
        env["MLFLOW_TRACKING_URI"] = tracking["tracking_uri"]
        env["MLFLOW_TRACKING_TOKEN"] = tracking["token"]
    return env


def run(experiment, config: dict, output, *, gpus: int | None = None, dry_run: bool = False) -> int:
    output = Path(output)
    plan = plan_for(experiment, config, output, gpus=gpus)
    (output / "launch_plan.json").write_text(plan.json())
    (output / "launch.sh").write_text("#!/bin/sh\nexec " + plan.shell() + "\n")
    if dry_run:
        return 0
    env = worker_environment()
    env.update(plan.env)
    argv = [sys.executable if t == "python" else t for t in plan.argv]
    proc = subprocess.run(argv, env=env)
    atomic_write_json(output / "launch_result.json", {"returncode": proc.returncode, "backend": plan.backend,
                                                      "metadata": dict(plan.metadata)})
    return proc.returncode
