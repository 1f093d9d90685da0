"""The preregistered repeated-data sweep for looped models: which (depth, recursions, weight decay) cells exist, what
they are called, and the launch plan that runs them -- fixed before any result is seen.

A cell is identified by a *reference depth* d (the depth axis of the protocol being transferred); the stored layer count
is ``5 d / 2`` (floor) and the hidden size ``128 * ceil(d / 8)`` (width and depth move together, rounded up to whole
multiples of 128 so that the expert-width ratio stays exact).  Every cell sees 100 M unique target tokens for 10 epochs.
``GRID`` lists the recursion counts per depth and ``WEIGHT_DECAYS`` the regularisation axis; the product is the whole
experiment.  ``cells()`` orders them: the anchor cell (d 8, K 2, wd 0.8) first, then the main wd-0.8 curves, then the
weight-decay controls.  A run may only be started for a cell of this list (``validate_cell``), under its canonical
name (``cell_name``).  ``write_plan`` derives the queue from a base plan's 128-wide "normal" run template: one run per
cell with its own port, output and qualification directory and the cell file passed as ``--sweep-cell``.
(Reference: src/archlab/automodel/loop_regularization.py:13-110.)
"""
from __future__ import annotations

import copy
import hashlib
import json
from pathlib import Path

from ..contracts.substrate import atomic_write_json

PROTOCOL_COMMIT = "9139c396957a57b6de9a1e7efe7e35a4a863f1a6"
WEIGHT_DECAYS = (0.05, 0.2, 0.4, 0.8, 1.2, 1.6)
GRID = {4: (6,), 6: (1, 2, 3, 4, 6), 8: (1, 2, 3, 4, 6, 8, 12), 10: (1, 2, 3, 4, 6, 8, 12), 12: (1, 2, 3, 4, 6, 8, 12), 14: (1, 2, 3, 4, 6, 8),
        16: (1, 2, 3), 18: (1,)}
ANCHOR = (8, 2, 0.8)
UNIQUE_TARGETS, EPOCHS = 100_000_000, 10
RUN_TOKEN_BUDGET, RUN_TOKEN_ALLOWANCE = 1_000_000_000, 10_000_000_000


def make_cell(depth: int, recursions: int, weight_decay: float) -> dict:
    return {"reference_depth": depth, "stored_layers": depth * 5 // 2, "hidden_size": 128 * -(-depth // 8), "recursions": recursions,
            "weight_decay": weight_decay, "unique_targets": UNIQUE_TARGETS, "epochs": EPOCHS, "reference_commit": PROTOCOL_COMMIT}


def _priority(cell: dict):
    key = (cell["reference_depth"], cell["recursions"], cell["weight_decay"])
    return (key != ANCHOR, cell["weight_decay"] != ANCHOR[2], *key)


def cells() -> list[dict]:
    every = [make_cell(d, k, wd) for d, loops in GRID.items() for k in loops for wd in WEIGHT_DECAYS]
    return sorted(every, key=_priority)


def validate_cell(cell: dict) -> None:
    d, k, wd = cell.get("reference_depth"), cell.get("recursions"), cell.get("weight_decay")
    if d not in GRID or k not in GRID[d] or wd not in WEIGHT_DECAYS or cell != make_cell(d, k, wd):
        raise ValueError("the cell differs from the preregistered repeated-data grid")


def cell_name(cell: dict) -> str:
    validate_cell(cell)
    return f"loop-d{cell['hidden_size']}-L{cell['stored_layers']}-K{cell['recursions']}-wd{str(cell['weight_decay']).replace('.', 'p')}"


def cells_sha256() -> str:
    return hashlib.sha256(json.dumps(cells(), sort_keys=True).encode()).hexdigest()


def write_plan(base_plan, *, source, commit: str, destination) -> dict:
    base = json.loads(Path(base_plan).read_text())
    root, source = Path(base["root"]), Path(source)
    template = next(r for r in base["runs"] if r["variant"] == "normal" and r["width"] == 128)
    environment = copy.deepcopy(base["environment"])
    environment["PYTHONPATH"] = ":".join([str(source), *environment.get("PYTHONPATH", "").split(":")[1:]])
    runs = []
    for index, cell in enumerate(cells()):
        name = cell_name(cell)
        cell_file = root / "sweep-cells" / f"{name}.json"
        cell_file.parent.mkdir(parents=True, exist_ok=True)
        atomic_write_json(cell_file, cell)
        runs.append({**template, "supplemental": True, "queue_index": index, "width": cell["hidden_size"], "source": str(source), "source_commit": commit,
                     "environment": environment, "master_port": 29000 + 2 * index, "qualification": str(root / f"qualification-{name}"),
                     "output": str(root / name), "extra_args": [*template.get("extra_args", []), "--sweep-cell", str(cell_file)],
                     "training_token_budget": RUN_TOKEN_BUDGET, "token_allowance": RUN_TOKEN_ALLOWANCE, "cell": cell})
    plan = {"format": "archlab-loop-repeated-data-sweep-v1", "runs": runs, "reference_commit": PROTOCOL_COMMIT, "cells_sha256": cells_sha256(),
            "planned_training_tokens": len(runs) * RUN_TOKEN_BUDGET, "token_allowance_per_run": RUN_TOKEN_ALLOWANCE,
            "scope": "repeated-data protocol transfer; anchor at reference depth 8 (20 stored layers, width 128); width and depth coupled, "
                     "widths rounded up to multiples of 128",
            "primary_compute_axis": "measured training GPU-seconds, excluding evaluation and checkpoint IO"}
    atomic_write_json(Path(destination), plan)
    return plan
