"""Strict, streamed loading of a released-name V4.1 checkpoint into one expert-parallel rank.

The checkpoint is a directory of one-tensor safetensors files with ``model.safetensors.index.json``; expert weights
are stored per expert (``...experts.<e>.w1|w2|w3.weight``), hashed tables optionally in row blocks (``<name>.rows.<r0>``).
Each rank reads ONLY what it owns:

* experts ``[rank * E / ep, (rank + 1) * E / ep)`` of every layer, written into the rank's slice of the stacked
  ``gate_and_up_projs`` (w1 | w3, transposed back) and ``down_projs`` (w2);
* for row-sharded tables, the contiguous row range of the table owner (defaults to the EP rank);
* every other tensor (replicated).

Nothing is loaded "best effort": a model parameter the checkpoint lacks, an owned expert part that is missing, a shard
file outside the checkpoint directory or a shape that does not fit is an error; tensors that are deliberately unused are
counted BY REASON (remote experts, remote table rows, inactive towers) so the report can be compared between ranks.
With ``require_verified_copy`` the directory must carry ``VERIFIED_COPY.json`` naming the index's SHA-256 (a staged copy
that was verified once is not re-hashed by every rank).  (Reference: src/archlab/automodel/deepseek_v41_loading.py:21-142;
the writer of this layout is ``ckpt.formats.export_v41_released``.)
"""
from __future__ import annotations

import hashlib
import json
import re
from collections import Counter
from pathlib import Path

import torch

from .formats import released_name

_EXPERT = re.compile(r"(?P<base>.*\.experts\.)(?P<e>\d+)\.(?P<part>w[123])\.weight")
_ROWS = re.compile(r"(?P<name>.*)\.rows\.(?P<r0>\d+)")
INACTIVE_PREFIXES = ("vision.", "aligner.", "mtp.")


def expert_range(n_experts: int, ep_rank: int, ep_size: int) -> range:
    if n_experts % ep_size:
        raise ValueError("the expert count must be divisible by the expert-parallel size")
    per = n_experts // ep_size
    return range(ep_rank * per, (ep_rank + 1) * per)


def _open(checkpoint: Path, file: str, key: str) -> torch.Tensor:
    from safetensors import safe_open

    if Path(file).name != file:
        raise ValueError("weight shards must be direct children of the checkpoint")
    with safe_open(str(checkpoint / file), framework="pt") as f:
        return f.get_tensor(key)


@torch.no_grad()
def load_released_ep(model: torch.nn.Module, checkpoint, *, ep_rank: int, ep_size: int, table_rank: int | None = None, table_size: int | None = None,
                     local_experts: bool = True, require_verified_copy: bool = False) -> dict:
    """``local_experts``: the model's stacked expert parameters hold only this rank's experts (shape[0] == E / ep);
    otherwise they hold all experts and only the owned slice is filled."""
    checkpoint = Path(checkpoint)
    table_rank, table_size = (ep_rank if table_rank is None else table_rank), (ep_size if table_size is None else table_size)
    if not 0 <= ep_rank < ep_size or not 0 <= table_rank < table_size:
        raise ValueError("invalid checkpoint loading geometry")
    raw = (checkpoint / "model.safetensors.index.json").read_bytes()
    if require_verified_copy:
        verified = json.loads((checkpoint / "VERIFIED_COPY.json").read_text())
        if verified.get("source_index_sha256") != hashlib.sha256(raw).hexdigest():
            raise ValueError("the index no longer matches the verified copy")
    mapping: dict[str, str] = json.loads(raw)["weight_map"]
    params = {released_name(n): (n, p) for n, p in model.named_parameters()}
    report, loaded = Counter(), set()
    stacks = {}                                                    # released base -> (gate_up param, down param, total experts)
    for key, (name, p) in params.items():
        if name.endswith(".experts.gate_and_up_projs"):
            stacks.setdefault(key.removesuffix("gate_and_up_projs"), {})["gate_up"] = p
        elif name.endswith(".experts.down_projs"):
            stacks.setdefault(key.removesuffix("down_projs"), {})["down"] = p
    totals = Counter()
    for key in mapping:
        m = _EXPERT.fullmatch(key)
        if m:
            totals[m["base"]] = max(totals[m["base"]], int(m["e"]) + 1)
    filled = Counter()
    for key, file in mapping.items():
        m = _EXPERT.fullmatch(key)
        if m and m["base"] in stacks:
            owned = expert_range(totals[m["base"]], ep_rank, ep_size)
            e = int(m["e"])
            if e not in owned:
                report["remote-expert-part"] += 1
                continue
            slot = e - owned.start if local_experts else e
            t = _open(checkpoint, file, key)
            stack = stacks[m["base"]]
            if m["part"] == "w2":
                stack["down"][slot].copy_(t.t())
            else:
                inter = stack["gate_up"].shape[-1] // 2
                half = slice(0, inter) if m["part"] == "w1" else slice(inter, 2 * inter)
                stack["gate_up"][slot][:, half].copy_(t.t())
            filled[(m["base"], e)] += 1
            report["owned-expert-part"] += 1
            continue
        r = _ROWS.fullmatch(key)
        if r and r["name"] in params:
            _, p = params[r["name"]]
            rows = p.shape[0]
            r0 = int(r["r0"])
            t = None
            if table_size > 1 and getattr(p, "row_sharded", False):
                per = -(-getattr(p, "global_rows", rows * table_size) // table_size)
                lo = table_rank * per
                t = _open(checkpoint, file, key)
                a, b = max(r0, lo), min(r0 + t.shape[0], lo + rows)
                if a >= b:
                    report["remote-table-rows"] += 1
                    continue
                p[a - lo:b - lo].copy_(t[a - r0:b - r0])
            else:
                t = _open(checkpoint, file, key)
                p[r0:r0 + t.shape[0]].copy_(t)
            loaded.add(r["name"])
            report["table-row-block"] += 1
            continue
        if key in params:
            _, p = params[key]
            t = _open(checkpoint, file, key)
            if t.shape != p.shape:
                raise ValueError(f"shape mismatch for {key}: checkpoint {tuple(t.shape)}, model {tuple(p.shape)}")
            p.copy_(t)
            loaded.add(key)
            report["replicated"] += 1
        elif key.startswith(INACTIVE_PREFIXES):
            report["inactive-tower"] += 1
        else:
            report["unused-other"] += 1
    for base, stack in stacks.items():
        owned = expert_range(totals[base], ep_rank, ep_size) if totals[base] else range(0)
        missing = [e for e in owned if filled[(base, e)] != 3]
        if missing or not totals[base]:
            raise ValueError(f"owned expert parts are missing for {base}: experts {missing[:8]}")
        loaded.update({base + "gate_and_up_projs", base + "down_projs"})
    absent = sorted(set(params) - loaded)
    if absent:
        raise ValueError(f"the checkpoint is missing model parameters: {absent[:10]}")
    return {"ep_rank": ep_rank, "ep_size": ep_size, "index_sha256": hashlib.sha256(raw).hexdigest(), "counts": dict(report), "parameters": len(params)}
