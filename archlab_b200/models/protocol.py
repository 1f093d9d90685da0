"""What every trainable model of this framework exposes to trainers, reports and qualification, and a mixin that
supplies the parts a model does not define itself.

    init_weights()                       materialises parameters and buffers (models build on the meta device)
    forward(ids, targets=None, ...)      logits, or a loss when targets are given
    num_scaling_params() -> dict         parameter counts by role; the values (without "total") sum to ``parameters()``
    estimate_flops() -> int              training FLOPs per token: 6 per matmul parameter + 12 * heads * head_dim * context per
                                         attention layer (embeddings and scalar gains excluded)
    estimate_executed_flops() -> int     the same with what really runs (sparse experts: only the routed share)
    set_training_step(step)              phase switches that depend on the step (dense warm-up of sparse attention ...)
    consume_training_metrics() -> dict   scalar metrics the last forward left behind; reading clears them
    get_architecture_state() -> dict     small, JSON-able mechanism state worth logging (expert load, phase)
    optimizer_contract() -> dict         which optimizer family owns which parameters; must cover every parameter once

(The reference states this protocol across its models: src/archlab/architectures/base.py:643-667,755-799,
dsa.py:424-429, qwen38_flash_next.py:1187-1200,1306-1312.)  ``ModelProtocol`` derives all of it from parameter names and
shapes and from ``self.config`` where that has the usual geometry fields; a model overrides what it knows better.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn

EMBEDDING_MARKERS = ("embed", "wte", "value_embeds", "tables", "engram")
HEAD_MARKERS = ("lm_head", "output_layer")
EXPERT_MARKERS = (".experts.",)


def _role(name: str, p: torch.Tensor) -> str:
    low = name.lower()
    if any(m in low for m in HEAD_MARKERS):
        return "lm_head"
    if any(m in low for m in EMBEDDING_MARKERS) and p.ndim >= 2:
        return "embeddings"
    if any(m in low for m in EXPERT_MARKERS) and p.ndim >= 2:
        return "expert_matrices"
    return "matrices" if p.ndim >= 2 else "scalars"


def _geometry(config) -> tuple[int, int, int, int]:
    """(attention layers, heads, head_dim, context) from the common config spellings; zeros when unknown."""
    get = lambda *names: next((getattr(config, n) for n in names if hasattr(config, n)), 0)
    layers = get("n_layer", "num_hidden_layers")
    heads = get("n_head", "n_heads", "num_attention_heads", "attention_heads")
    head_dim = get("head_dim", "attention_head_dim") or (get("n_embd", "hidden_size") // heads if heads else 0)
    context = get("sequence_len", "max_position_embeddings", "max_seq_len")
    interval = get("full_attention_interval")
    if interval:                                                    # hybrid stacks: only every k-th layer is softmax attention
        layers = layers // interval
    return int(layers), int(heads), int(head_dim), int(context)


class ModelProtocol:
    def num_scaling_params(self) -> dict[str, int]:
        out: dict[str, int] = {}
        for name, p in self.named_parameters():
            role = _role(name, p)
            out[role] = out.get(role, 0) + p.numel()
        out["total"] = sum(out.values())
        return out

    def _routed_share(self) -> float:
        c = getattr(self, "config", None)
        total = next((getattr(c, n) for n in ("n_routed_experts", "n_experts") if c is not None and getattr(c, n, 0)), 0)
        active = getattr(c, "experts_top_k", 0) if c is not None else 0
        return active / total if total and active else 1.0

    def _flops(self, expert_share: float) -> int:
        counts = self.num_scaling_params()
        matmul = counts.get("matrices", 0) + counts.get("lm_head", 0) + expert_share * counts.get("expert_matrices", 0)
        layers, heads, head_dim, context = _geometry(getattr(self, "config", None))
        return int(6 * matmul + 12 * layers * heads * head_dim * context)

    def estimate_flops(self) -> int:
        return self._flops(1.0)

    def estimate_executed_flops(self) -> int:
        return self._flops(self._routed_share())

    def set_training_step(self, step: int) -> None:
        self.step = int(step)
        for module in self.modules():
            if module is not self and hasattr(module, "set_step") and callable(module.set_step):
                module.set_step(int(step))

    def consume_training_metrics(self) -> dict[str, float]:
        out = {}
        own = getattr(self, "last_loss_metrics", None)
        if own:
            out.update({k: float(v) for k, v in own.items() if torch.is_tensor(v) and v.numel() == 1 or isinstance(v, (int, float))})
            self.last_loss_metrics = {}
        aux = [float(torch.as_tensor(m.last_metrics["aux_loss"]).detach()) for m in self.modules() if isinstance(getattr(m, "last_metrics", None), dict) and "aux_loss" in m.last_metrics]
        if aux:
            out["router aux loss"] = sum(aux) / len(aux)
        return out

    def get_architecture_state(self) -> dict:
        state = {"step": int(getattr(self, "step", 0))}
        loads = [m._cumulative_expert_load for m in self.modules() if getattr(m, "_cumulative_expert_load", None) is not None]
        if loads:
            share = torch.stack([l / l.sum().clamp_min(1) for l in loads])
            state["expert_load"] = {"layers": len(loads), "max_share": float(share.max()), "dead_experts": int((share == 0).sum()),
                                    "cv": float((share.std(-1) / share.mean(-1).clamp_min(1e-12)).mean())}
        return state

    def optimizer_contract(self) -> dict:
        """Matrices inside the trunk go to the matrix optimizer (Muon family), embeddings / head / scalars to AdamW."""
        groups: dict[str, list[str]] = {"muon": [], "adamw": []}
        for name, p in self.named_parameters():
            groups["muon" if _role(name, p) in ("matrices", "expert_matrices") and p.ndim >= 2 else "adamw"].append(name)
        names = [n for g in groups.values() for n in g]
        if len(names) != len(set(names)) or len(names) != sum(1 for _ in self.parameters()):
            raise AssertionError("the optimizer contract must cover every parameter exactly once")
        return groups


def attach_protocol(cls: type) -> type:
    """Adds the protocol's methods to ``cls`` where it does not define them itself."""
    for name, member in vars(ModelProtocol).items():
        if callable(member) and not name.startswith("__") and name not in cls.__dict__ and not any(name in vars(b) for b in cls.__mro__[1:] if b not in (nn.Module, object)):
            setattr(cls, name, member)
    return cls


def check_protocol(model: nn.Module) -> dict:
    """Raises if the model breaks the protocol; returns the headline numbers."""
    counts = model.num_scaling_params()
    total = sum(p.numel() for p in model.parameters())
    if sum(v for k, v in counts.items() if k != "total") != total or counts.get("total", total) != total:
        raise AssertionError("num_scaling_params() does not sum to the model's parameters")
    flops, executed = model.estimate_flops(), model.estimate_executed_flops() if hasattr(model, "estimate_executed_flops") else None
    if flops <= 0 or (executed is not None and not 0 < executed <= flops):
        raise AssertionError("FLOP estimates must be positive and executed <= dense")
    contract = model.optimizer_contract()
    named = [n for g in contract.values() for n in (g if isinstance(g, list) else [])]
    if named and sorted(named) != sorted(n for n, _ in model.named_parameters()):
        raise AssertionError("optimizer_contract() does not cover every parameter exactly once")
    model.set_training_step(3)
    json_state = model.get_architecture_state()
    import json

    json.dumps(json_state)
    if not isinstance(model.consume_training_metrics(), dict):
        raise AssertionError("consume_training_metrics() must return a dict")
    return {"parameters": total, "flops_per_token": flops, "executed_flops_per_token": executed}
