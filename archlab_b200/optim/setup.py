"""Parameter grouping and schedules of the speedrun recipe.

Grouping follows src/archlab/optimizers/speedrun.py:758-842 (``_base_parameter_groups``) and
:1077-1164 (``setup_model_optimizer``): AdamW for lm_head / wte / value embeddings / scalars with
learning rates scaled by ``(d_model / 768) ** -0.5``, Muon for every 2-D trunk matrix with one
group per distinct shape.  Schedules follow src/archlab/speedrun/base_train.py:1556-1590.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..parallel import collectives as coll
from .dist_muon import DistMuonAdamW
from .muon import MuonAdamW

MATRIX_MODES = {"normuon", "muonh", "muoneqh-half", "muoneqh-quarter", "adamh"}


def adamw_group(params, lr, betas, weight_decay, **meta) -> dict:
    return {"kind": "adamw", "params": list(params), "lr": lr, "betas": betas, "eps": 1e-10,
            "weight_decay": weight_decay, **meta}


def muon_groups(params, matrix_lr, weight_decay) -> list[dict]:
    params = list(params)
    return [
        {"kind": "muon", "params": [p for p in params if p.shape == shape], "lr": matrix_lr,
         "momentum": 0.95, "ns_steps": 5, "beta2": 0.9, "weight_decay": weight_decay}
        for shape in sorted({p.shape for p in params})
    ]


def base_parameter_groups(model, *, unembedding_lr, embedding_lr, matrix_lr, weight_decay, scalar_lr):
    scale = (model.config.n_embd / 768) ** -0.5
    trunk = list(model.transformer.h.parameters())
    matrices = [p for p in trunk if p.ndim == 2]
    other = [p for p in trunk if p.ndim != 2]
    groups = [
        adamw_group(model.lm_head.parameters(), unembedding_lr * scale, (0.8, 0.96), 0.01),
        adamw_group(model.transformer.wte.parameters(), embedding_lr * scale, (0.8, 0.995), 0.001),
        adamw_group(model.value_embeds.parameters(), embedding_lr * scale * 0.5, (0.8, 0.995), 0.01),
        adamw_group([model.resid_lambdas], scalar_lr * 0.01, (0.8, 0.95), 0.05),
        adamw_group([model.x0_lambdas], scalar_lr, (0.96, 0.95), 0.0),
        adamw_group([model.smear_gate.weight, model.smear_lambda, model.backout_lambda], 0.2, (0.8, 0.95), 0.0),
    ]
    if other:
        groups.append(adamw_group(other, scalar_lr * 0.01, (0.8, 0.95), 0.0))
    groups.extend(muon_groups(matrices, matrix_lr, weight_decay))
    return [g for g in groups if g["params"]]


def setup_model_optimizer(model, *, unembedding_lr=0.004, embedding_lr=0.2, matrix_lr=0.02, weight_decay=0.0,
                          scalar_lr=0.5, distributed: bool | None = None, matrix_optimizer: str = "normuon",
                          adam_update_every: int = 1, cautious_adam_weight_decay: bool = False,
                          group_builder=None, process_group=None):
    if matrix_optimizer not in MATRIX_MODES:
        raise ValueError(f"unknown matrix_optimizer={matrix_optimizer!r}")
    if adam_update_every < 1:
        raise ValueError("adam_update_every must be positive")
    builder = group_builder or getattr(model, "parameter_groups", None) or base_parameter_groups
    if builder is base_parameter_groups:
        groups = builder(model, unembedding_lr=unembedding_lr, embedding_lr=embedding_lr, matrix_lr=matrix_lr,
                         weight_decay=weight_decay, scalar_lr=scalar_lr)
    else:
        groups = builder(unembedding_lr=unembedding_lr, embedding_lr=embedding_lr, matrix_lr=matrix_lr,
                         weight_decay=weight_decay, scalar_lr=scalar_lr)
    for g in groups:
        if g["kind"] == "adamw":
            g["update_every"] = adam_update_every
            g["cautious_weight_decay"] = cautious_adam_weight_decay
        elif g["kind"] == "muon":
            g["hyperball"] = matrix_optimizer.startswith("muon") and matrix_optimizer != "normuon"
            g["equilibrate_exponent"] = {"muoneqh-half": -0.5, "muoneqh-quarter": -0.25}.get(matrix_optimizer, 0.0)
            if matrix_optimizer == "adamh":
                g.update(kind="adamh", betas=(0.9, 0.95), eps=1e-10, weight_decay=0.0)
    ids = [id(p) for g in groups for p in g["params"]]
    if len(ids) != len(set(ids)) or set(ids) != {id(p) for p in model.parameters()}:
        raise RuntimeError("optimizer parameter grouping mismatch")
    if distributed is None:
        distributed = coll.is_dist() and coll.world_size(process_group) > 1
    if distributed and matrix_optimizer == "adamh":
        raise NotImplementedError("AdamH recipe is not implemented for the distributed optimizer")
    opt = DistMuonAdamW(groups, group=process_group) if distributed else MuonAdamW(groups)
    for g in opt.param_groups:
        g.setdefault("initial_lr", g["lr"])
    return opt


@dataclass
class Schedule:
    num_iterations: int
    warmup_steps: int = 40
    warmdown_ratio: float = 0.65
    final_lr_frac: float = 0.05
    weight_decay: float = 0.28

    def lr_multiplier(self, it: int) -> float:
        warmdown = round(self.warmdown_ratio * self.num_iterations)
        if it < self.warmup_steps:
            return (it + 1) / self.warmup_steps
        if it <= self.num_iterations - warmdown:
            return 1.0
        progress = (self.num_iterations - it) / warmdown
        return progress + (1 - progress) * self.final_lr_frac

    def muon_momentum(self, it: int) -> float:
        warmdown = round(self.warmdown_ratio * self.num_iterations)
        start = self.num_iterations - warmdown
        if it < 400:
            f = it / 400
            return (1 - f) * 0.85 + f * 0.97
        if it >= start and warmdown > 0:
            pr = (it - start) / warmdown
            return 0.97 * (1 - pr) + 0.90 * pr
        return 0.97

    def muon_weight_decay(self, it: int) -> float:
        return self.weight_decay * 0.5 * (1 + math.cos(math.pi * it / self.num_iterations))

    def apply(self, optimizer: torch.optim.Optimizer, it: int) -> None:
        lrm = self.lr_multiplier(it)
        for g in optimizer.param_groups:
            g["lr"] = g["initial_lr"] * lrm
            if g["kind"] == "muon":
                g["momentum"] = self.muon_momentum(it)
                g["weight_decay"] = self.muon_weight_decay(it)
