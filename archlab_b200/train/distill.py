"""Three-stage conversion of a teacher into a student with replaced token mixers.

Stage 1 (latent matching): the teacher runs once per batch; forward hooks record, for every replaced
layer, the mixer's input and output.  Each replacement mixer is fitted to reproduce the output from
the SAME input (independent squared reconstruction losses, summed over layers), so no gradient flows
between layers and the backbone stays frozen.
Stage 2 (forward KL): the composed student is trained against the teacher's next-token distribution,
KL(teacher || student), evaluated in token chunks so that the [tokens, vocab] logits of both models
never exist at once; replaced mixers and backbone use two learning rates.
Stage 3 (on-policy reverse KL): the student continues prompts itself; KL(student || teacher) is taken
on the generated positions.  The generation horizon doubles whenever the smoothed reverse KL stops
improving without having diverged; the learning rate follows a token-parameterised
warm-up / stable / decay schedule.

Checkpoints carry model + optimizer + every rank's RNG + a fingerprint of the run contract, and refuse
to load under a different fingerprint.  Mirrors src/archlab/training/latent_match.py:222-437,
stage2_distill.py:206-447 and stage3_onpolicy.py:62-620 in behaviour; models are plain callables
``model(ids) -> logits`` with ``nn.Module`` mixers, so every piece runs on CPU in tests.
"""
from __future__ import annotations

import hashlib
import json
import math
import os
from contextlib import contextmanager
from dataclasses import dataclass
from pathlib import Path

import torch
import torch.nn as nn
import torch.nn.functional as F


# ------------------------------------------------------------------------------------------------
# schedules
# ------------------------------------------------------------------------------------------------
def cosine_lr(step: int, total: int, peak: float, warmup_fraction: float, final_fraction: float) -> float:
    warm = int(total * warmup_fraction)
    if warm and step < warm:
        return peak * (step + 1) / warm
    prog = (step - warm) / max(1, total - warm - 1)
    return peak * (final_fraction + (1 - final_fraction) * 0.5 * (1 + math.cos(math.pi * prog)))


def wsd_lr(tokens_done: int, total_tokens: int, peak: float, warmup_fraction: float = 0.03, decay_fraction: float = 0.10,
           final_fraction: float = 0.10) -> float:
    if total_tokens <= 0 or tokens_done < 0:
        raise ValueError("token counts must be a positive total and non-negative progress")
    if not (0 <= warmup_fraction < 1 and 0 <= decay_fraction < 1 and warmup_fraction + decay_fraction <= 1):
        raise ValueError("invalid warm-up / decay fractions")
    if not (0 <= final_fraction <= 1 and math.isfinite(peak) and peak > 0):
        raise ValueError("invalid peak or final learning rate")
    prog = min(float(total_tokens), float(max(1, tokens_done)))
    warm, decay_start = total_tokens * warmup_fraction, total_tokens * (1 - decay_fraction)
    if warm > 0 and prog < warm:
        return peak * prog / warm
    if decay_fraction > 0 and prog > decay_start:
        ratio = min(1.0, (prog - decay_start) / max(1e-9, total_tokens - decay_start))
        return peak * (1 - ratio * (1 - final_fraction))
    return peak


@dataclass
class HorizonCurriculum:
    """Generation length doubles on a plateau of the smoothed reverse KL that has not diverged."""
    gen_tokens: int
    phase: int = 0
    smoothed: float | None = None
    best: float | None = None
    phase_start: float | None = None
    stale: int = 0

    def update(self, reverse_kl: float, *, max_gen_tokens: int, ema: float = 0.2, improvement: float = 0.02,
               plateau_steps: int = 30, max_divergence: float = 0.05) -> bool:
        if not math.isfinite(reverse_kl):
            raise FloatingPointError("non-finite reverse KL")
        if self.phase_start is None:
            self.phase_start = reverse_kl if self.smoothed is None else self.smoothed
        self.smoothed = reverse_kl if self.smoothed is None else (1 - ema) * self.smoothed + ema * reverse_kl
        if self.best is None or self.smoothed <= self.best * (1 - improvement):
            self.best, self.stale = self.smoothed, 0
        else:
            self.stale += 1
        ceiling = max(self.phase_start * (1 + max_divergence), self.phase_start + 1e-6)
        if self.stale >= plateau_steps and self.gen_tokens < max_gen_tokens and self.smoothed <= ceiling:
            self.gen_tokens = min(max_gen_tokens, self.gen_tokens * 2)
            self.phase += 1
            self.smoothed = self.best = self.phase_start = None
            self.stale = 0
            return True
        return False


def horizons(min_tokens: int, max_tokens: int) -> tuple[int, ...]:
    if min_tokens < 1 or max_tokens < min_tokens:
        raise ValueError("invalid horizon bounds")
    out = [min_tokens]
    while out[-1] < max_tokens:
        if out[-1] * 2 > max_tokens:
            raise ValueError("the largest horizon must be a power-of-two multiple of the smallest")
        out.append(out[-1] * 2)
    return tuple(out)


# ------------------------------------------------------------------------------------------------
# stage 1: latent matching
# ------------------------------------------------------------------------------------------------
@contextmanager
def capture(mixers: dict[int, nn.Module]):
    """Record (input hidden states, extra kwargs, output) of each teacher mixer during one forward."""
    store, handles = {}, []
    for idx, m in mixers.items():
        def hook(mod, args, kwargs, out, idx=idx):
            hidden = args[0] if args else kwargs["hidden_states"]
            out0 = out[0] if isinstance(out, tuple) else out
            store[idx] = (hidden.detach(), {k: v for k, v in kwargs.items() if k != "hidden_states"}, out0.detach())
        handles.append(m.register_forward_hook(hook, with_kwargs=True))
    try:
        yield store
    finally:
        for h in handles:
            h.remove()


def reconstruction_loss(output, target, kind: str = "mse"):
    if output.shape != target.shape or output.ndim != 3:
        raise ValueError("mixer outputs must both be [batch, tokens, hidden]")
    err = (output.float() - target.detach().float()).square().mean(dim=(1, 2))
    if kind == "normalized_mse":
        err = err / target.detach().float().square().mean(dim=(1, 2)).clamp_min(1e-12)
    elif kind != "mse":
        raise ValueError("unknown reconstruction loss")
    return err.mean()


def latent_match_step(teacher, mixers: dict[int, nn.Module], switches: dict[int, nn.Module], optimizer, ids, *,
                      loss_kind: str = "mse", clip_norm: float = 1.0) -> dict:
    with torch.no_grad(), capture(mixers) as store:
        teacher(ids)
    if set(store) != set(switches):
        raise ValueError("the teacher did not visit exactly the replaced layers")
    optimizer.zero_grad(set_to_none=True)
    per_layer, total = {}, 0.0
    for idx, sw in switches.items():
        hidden, kwargs, target = store[idx]
        out = sw(hidden, **kwargs)
        out = out[0] if isinstance(out, tuple) else out
        loss = reconstruction_loss(out, target, loss_kind)
        loss.backward()                                          # layers are independent: no graph is shared
        per_layer[idx] = float(loss.detach())
        total += per_layer[idx]
    params = [p for sw in switches.values() for p in sw.parameters() if p.grad is not None]
    gnorm = float(torch.nn.utils.clip_grad_norm_(params, clip_norm)) if params else 0.0
    if not math.isfinite(total) or not math.isfinite(gnorm):
        raise FloatingPointError("non-finite latent-matching loss or gradient")
    optimizer.step()
    return {"loss": total, "per_layer": per_layer, "grad_norm": gnorm}


# ------------------------------------------------------------------------------------------------
# stage 2 / 3: chunked KL
# ------------------------------------------------------------------------------------------------
def two_timescale_optimizer(student: nn.Module, switches: dict[int, nn.Module], *, lr: float, backbone_lr_ratio: float,
                            weight_decay: float = 0.0):
    fast = {id(p) for sw in switches.values() for p in sw.parameters()}
    groups = [{"params": [p for p in student.parameters() if id(p) in fast and p.requires_grad], "lr": lr, "role": "switch"},
              {"params": [p for p in student.parameters() if id(p) not in fast and p.requires_grad],
               "lr": lr * backbone_lr_ratio, "role": "backbone"}]
    groups = [g for g in groups if g["params"]]
    for g in groups:
        g["base_lr"] = g["lr"]
    return torch.optim.AdamW(groups, betas=(0.9, 0.95), weight_decay=weight_decay)


def _kl_rows(p_logits, q_logits):
    """KL(P || Q) per row from logits, in fp32."""
    lp, lq = F.log_softmax(p_logits.float(), -1), F.log_softmax(q_logits.float(), -1)
    return (lp.exp() * (lp - lq)).sum(-1)


def chunked_kl_step(teacher_hidden_fn, student_hidden_fn, teacher_head, student_head, ids, mask, *, direction: str,
                    chunk_tokens: int = 128, scale: float = 1.0) -> float:
    """Backward of mean KL over the masked positions without materialising full-vocabulary logits.

    ``*_hidden_fn(ids) -> [B, T, C]`` give final hidden states; ``*_head(h) -> logits``.  The student's
    hidden states keep their graph; each chunk's head + KL is differentiated immediately into the
    hidden-state gradient, which is sent back through the trunk once.  ``direction`` is ``forward``
    (KL(teacher || student)) or ``reverse`` (KL(student || teacher))."""
    with torch.no_grad():
        th = teacher_hidden_fn(ids)
    sh = student_hidden_fn(ids)
    flat_s, flat_t, flat_m = sh.flatten(0, 1), th.flatten(0, 1), mask.flatten().bool()
    n = int(flat_m.sum())
    if n == 0:
        raise ValueError("no supervised positions")
    leaf = flat_s.detach().requires_grad_(True)
    total = 0.0
    for s in range(0, leaf.size(0), chunk_tokens):
        m = flat_m[s:s + chunk_tokens]
        if not bool(m.any()):
            continue
        sl = student_head(leaf[s:s + chunk_tokens][m])
        with torch.no_grad():
            tl = teacher_head(flat_t[s:s + chunk_tokens][m])
        kl = _kl_rows(tl, sl) if direction == "forward" else _kl_rows(sl, tl)
        part = kl.sum() * (scale / n)
        part.backward()                                           # head parameters and `leaf.grad` accumulate
        total += float(kl.detach().sum())
    flat_s.backward(leaf.grad)
    return total / n


@torch.no_grad()
def rollout(student_logits_fn, prompts: torch.Tensor, gen_tokens: int, *, temperature: float = 1.0,
            generator: torch.Generator | None = None):
    """Sample ``gen_tokens`` continuations; returns (ids [B, P + G], mask of generated positions whose
    NEXT-token distribution is supervised, i.e. positions P-1 .. P+G-2)."""
    ids = prompts.clone()
    for _ in range(gen_tokens):
        logits = student_logits_fn(ids)[:, -1].float() / max(temperature, 1e-6)
        nxt = torch.multinomial(F.softmax(logits, -1), 1, generator=generator)
        ids = torch.cat([ids, nxt], 1)
    mask = torch.zeros_like(ids, dtype=torch.bool)
    mask[:, prompts.size(1) - 1: ids.size(1) - 1] = True
    return ids, mask


# ------------------------------------------------------------------------------------------------
# checkpoints
# ------------------------------------------------------------------------------------------------
def contract_hash(contract: dict) -> str:
    return hashlib.sha256(json.dumps(contract, sort_keys=True, separators=(",", ":")).encode()).hexdigest()


def rank_rng_state(device: torch.device | None = None) -> dict:
    out = {"torch": torch.get_rng_state()}
    if device is not None and device.type == "cuda":
        out["cuda"] = torch.cuda.get_rng_state(device)
    return out


def restore_rank_rng(saved: dict, device: torch.device | None = None) -> None:
    torch.set_rng_state(saved["torch"])
    if device is not None and device.type == "cuda" and "cuda" in saved:
        torch.cuda.set_rng_state(saved["cuda"], device)


def atomic_torch_save(path: Path, state: dict) -> Path:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_name(f".{path.name}.{os.getpid()}.tmp")
    torch.save(state, tmp)
    os.replace(tmp, path)
    return path


def save_stage_checkpoint(output: Path, step: int, modules: dict[str, nn.Module], optimizer, rngs: list[dict], fingerprint: str,
                          extra: dict | None = None) -> Path:
    """``rngs`` holds one entry per rank (gathered by the caller); written by rank 0."""
    state = {"step": step, "fingerprint": fingerprint, "modules": {k: m.state_dict() for k, m in modules.items()},
             "optimizer": optimizer.state_dict(), "rng": rngs, "extra": extra or {}}
    return atomic_torch_save(Path(output) / f"step-{step:07d}.pt", state)


def load_stage_checkpoint(path: Path, modules: dict[str, nn.Module], optimizer, fingerprint: str, *, rank: int = 0, world: int = 1,
                          device: torch.device | None = None) -> dict:
    state = torch.load(path, map_location="cpu", weights_only=False)
    if state["fingerprint"] != fingerprint:
        raise ValueError("checkpoint belongs to a different run contract")
    if len(state["rng"]) != world:
        raise ValueError("checkpoint was written by a different world size")
    for k, m in modules.items():
        m.load_state_dict(state["modules"][k])
    optimizer.load_state_dict(state["optimizer"])
    restore_rank_rng(state["rng"][rank], device)
    return {"step": state["step"], "extra": state["extra"]}
