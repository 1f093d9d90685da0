"""Adapter warm-up followed by full-weight training without losing the adapter's optimizer history.

Phase 1 trains only the adapters with a plain AdamW.  Phase 2 unfreezes the backbone: its low-precision parameters get
fp32 master copies and fp32 moments (``MasterAdamW``), while the adapters keep THEIR optimizer object, moments and step
counts.  ``SplitAdamW`` composes the two; its state dict carries both parts under a format tag, and it also accepts a
plain phase-1 AdamW state (a checkpoint written before the backbone had any training history loads into the adapter
half only).

``warmup_learning_rates`` keeps two clocks: the adapter schedule continues from the run's start (linear warm-up, cosine
to 10 % over the run's token target), the backbone schedule starts at the step / token count at which full-weight
training began and has its own warm-up and its own cosine over the REMAINING tokens.
(Reference: src/archlab/optimizers/limite_warmup.py:12-96.)
"""
from __future__ import annotations

import math

import torch

FORMAT = "archlab-split-adamw-v1"


def _cosine_floor(progress: float, floor: float = 0.1) -> float:
    return floor + (1 - floor) * 0.5 * (1 + math.cos(math.pi * progress))


def warmup_learning_rates(step: int, tokens: int, schedule: dict) -> tuple[float, float]:
    target = schedule["target_tokens"]
    start_step, start_tokens = schedule["full_weight_start_step"], schedule["full_weight_start_tokens"]
    adapter = schedule["adapter_peak_lr"] * min(1.0, (step + 1) / schedule["adapter_warmup_steps"]) * _cosine_floor(tokens / target)
    backbone = (schedule["backbone_peak_lr"] * min(1.0, (step - start_step + 1) / schedule["backbone_warmup_steps"])
                * _cosine_floor((tokens - start_tokens) / (target - start_tokens)))
    return adapter, backbone


class MasterAdamW(torch.optim.Optimizer):
    """AdamW whose update runs on fp32 master weights and fp32 moments; the model's (bf16 / fp16) parameters are the
    rounded copy.  fp32 parameters are their own masters."""

    def __init__(self, params, lr=1e-5, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self):
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["master"] = p.detach().float().clone() if p.dtype != torch.float32 else None
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                st["step"] += 1
                w = st["master"] if st["master"] is not None else p
                g = p.grad.float()
                st["exp_avg"].lerp_(g, 1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(g, g, value=1 - b2)
                w.mul_(1 - group["lr"] * group["weight_decay"])
                denom = (st["exp_avg_sq"] / (1 - b2 ** st["step"])).sqrt_().add_(group["eps"])
                w.addcdiv_(st["exp_avg"], denom, value=-group["lr"] / (1 - b1 ** st["step"]))
                if st["master"] is not None:
                    p.copy_(w)


    def load_state_dict(self, state_dict: dict) -> None:
        """The base class casts floating-point state to each parameter's dtype, which would round the fp32 masters and
        moments of bf16 parameters; they are restored from the saved tensors afterwards."""
        super().load_state_dict(state_dict)
        ordered = [p for g in self.param_groups for p in g["params"]]
        saved_ids = [i for g in state_dict["param_groups"] for i in g["params"]]
        for p, i in zip(ordered, saved_ids):
            for key, value in state_dict["state"].get(i, {}).items():
                if torch.is_tensor(value) and value.is_floating_point():
                    self.state[p][key] = value.detach().to(device=p.device, dtype=torch.float32).clone()


class SplitAdamW:
    def __init__(self, adapter: torch.optim.Optimizer, backbone: torch.optim.Optimizer):
        self.adapter, self.backbone = adapter, backbone

    @property
    def param_groups(self):
        return self.adapter.param_groups + self.backbone.param_groups

    def set_learning_rates(self, adapter_lr: float, backbone_lr: float) -> None:
        for g in self.adapter.param_groups:
            g["lr"] = adapter_lr
        for g in self.backbone.param_groups:
            g["lr"] = backbone_lr

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.adapter.zero_grad(set_to_none=set_to_none)
        self.backbone.zero_grad(set_to_none=set_to_none)

    def step(self) -> None:
        self.adapter.step()
        self.backbone.step()

    def state_dict(self) -> dict:
        return {"format": FORMAT, "adapter": self.adapter.state_dict(), "backbone": self.backbone.state_dict()}

    def load_state_dict(self, state: dict) -> None:
        if state.get("format") == FORMAT:
            self.adapter.load_state_dict(state["adapter"])
            self.backbone.load_state_dict(state["backbone"])
        elif "state" in state and "param_groups" in state:          # a phase-1 checkpoint: the backbone has no history yet
            self.adapter.load_state_dict(state)
        else:
            raise ValueError("unsupported warm-up optimizer state")


def build_warmup_optimizer(adapter_parameters, backbone_parameters=(), *, lr=1e-4, backbone_lr=1e-5, betas=(0.9, 0.95), weight_decay=0.0):
    """Phase 1 (no trainable backbone parameters): the adapter AdamW alone.  Phase 2: the composition."""
    adapter_parameters = list(adapter_parameters)
    adapter = torch.optim.AdamW(adapter_parameters, lr=lr, betas=betas, weight_decay=weight_decay)
    ids = {id(p) for p in adapter_parameters}
    backbone_parameters = [p for p in backbone_parameters if p.requires_grad and id(p) not in ids]
    if not backbone_parameters:
        return adapter
    return SplitAdamW(adapter, MasterAdamW(backbone_parameters, lr=backbone_lr, betas=betas, weight_decay=weight_decay))
