"""The three recovery stages after a mechanism switch, as resumable runs that chain through their checkpoints.

Stage 1  latent matching: each replacement mixer is fitted, layer by layer, to reproduce the frozen teacher's mixer on
         the teacher's own inputs (cosine schedule).  Output: the switches.
Stage 2  composed forward KL: the switches are installed in the student; KL(teacher || student) over teacher-forced
         windows, switches at the full rate and the backbone at a fraction of it (two time scales), learning rate
         parameterised by *tokens* (warm-up / stable / decay).  Output: the composed student.
Stage 3  on-policy reverse KL: the student continues prompts itself and is pulled towards the teacher on its own
         trajectories, KL(student || teacher) on generated positions only, with an optional forward-KL anchor on
         teacher-forced data; the generation horizon doubles when the smoothed reverse KL plateaus without diverging.

Every stage is described by a config dataclass, fingerprints its contract (config + lineage: the fingerprint and the
checkpoint hash of the stage it starts from), saves atomically, resumes only into the same contract, and refuses to
start from a checkpoint of the wrong stage.  The reference runs the same three stages as three scripts
(src/archlab/training/distill.py, stage2_distill.py:50-560, stage3_onpolicy.py:62-760); the math lives in
``train.distill``, this module is the run logic.

A *bundle* supplies the models: ``teacher`` and ``student`` (``hidden(ids)``, ``head`` callable on hidden states),
``teacher_mixers`` / ``student_sites`` (layer -> module to replace) and ``make_switch(layer)``.
"""
from __future__ import annotations

import hashlib
import json
import math
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Callable

import torch
import torch.nn as nn

from . import distill as D


@dataclass
class Bundle:
    teacher: nn.Module
    student: nn.Module
    teacher_mixers: dict[int, nn.Module]
    install: Callable[[nn.Module, int, nn.Module], None]      # (student, layer, switch): put the switch in place
    make_switch: Callable[[int], nn.Module]
    teacher_head: Callable = None
    student_head: Callable = None

    def __post_init__(self):
        self.teacher_head = self.teacher_head or self.teacher.head
        self.student_head = self.student_head or self.student.head
        for p in self.teacher.parameters():
            p.requires_grad_(False)


@dataclass(frozen=True)
class Stage1Config:
    steps: int = 200
    lr: float = 3e-3
    warmup_fraction: float = 0.05
    final_lr_fraction: float = 0.1
    loss: str = "normalized_mse"
    save_every: int = 0
    seed: int = 0


@dataclass(frozen=True)
class Stage2Config:
    total_tokens: int = 20000
    lr: float = 1e-3
    backbone_lr_ratio: float = 0.1
    chunk_tokens: int = 128
    clip_norm: float = 1.0
    save_every: int = 0
    seed: int = 0


@dataclass(frozen=True)
class Stage3Config:
    total_tokens: int = 20000
    lr: float = 5e-4
    backbone_lr_ratio: float = 0.1
    temperature: float = 1.0
    min_gen_tokens: int = 4
    max_gen_tokens: int = 16
    plateau_steps: int = 10
    anchor_kl_weight: float = 0.0
    chunk_tokens: int = 128
    clip_norm: float = 1.0
    save_every: int = 0
    seed: int = 0

    def __post_init__(self):
        D.horizons(self.min_gen_tokens, self.max_gen_tokens)          # refuses bounds that doubling cannot reach
        if self.temperature <= 0 or self.anchor_kl_weight < 0:
            raise ValueError("temperature must be positive and the anchor weight non-negative")


def file_sha256(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for block in iter(lambda: f.read(1 << 20), b""):
            h.update(block)
    return h.hexdigest()


class _StageRun:
    """Directory, contract, metrics ledger, checkpoints and resume of one stage."""

    def __init__(self, stage: int, output, config, lineage: dict | None):
        self.stage = stage
        self.dir = Path(output)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.config = config
        self.contract = {"stage": self.stage, "config": asdict(config), "lineage": lineage}
        self.fingerprint = D.contract_hash(self.contract)
        contract_file = self.dir / "RUN_CONTRACT.json"
        if contract_file.exists():
            if json.loads(contract_file.read_text())["fingerprint"] != self.fingerprint:
                raise ValueError(f"{self.dir} holds a run with a different contract")
        else:
            contract_file.write_text(json.dumps({**self.contract, "fingerprint": self.fingerprint}, indent=2, sort_keys=True) + "\n")
        self.ledger = self.dir / "metrics.jsonl"

    def log(self, row: dict) -> None:
        with self.ledger.open("a") as f:
            f.write(json.dumps(row) + "\n")

    def newest(self) -> Path | None:
        found = sorted(self.dir.glob("step-*.pt"))
        return found[-1] if found else None

    def save(self, step: int, modules: dict, optimizer, extra: dict) -> Path:
        return D.save_stage_checkpoint(self.dir, step, modules, optimizer, [D.rank_rng_state()], self.fingerprint,
                                       {"stage": self.stage, **extra})

    def resume(self, modules: dict, optimizer) -> dict | None:
        path = self.newest()
        return None if path is None else D.load_stage_checkpoint(path, modules, optimizer, self.fingerprint)

    def finish(self, step: int, modules: dict, optimizer, extra: dict) -> dict:
        path = self.save(step, modules, optimizer, {**extra, "final": True})
        receipt = {"stage": self.stage, "fingerprint": self.fingerprint, "checkpoint": path.name, "checkpoint_sha256": file_sha256(path),
                   "steps": step, **extra}
        (self.dir / "COMPLETE.json").write_text(json.dumps(receipt, indent=2, sort_keys=True) + "\n")
        return receipt


def lineage_of(previous_dir, expected_stage: int) -> tuple[dict, dict]:
    """(lineage entry, checkpoint state) of a finished earlier stage; refuses unfinished runs, the wrong stage and a
    checkpoint that no longer matches its receipt."""
    previous = Path(previous_dir)
    receipt_file = previous / "COMPLETE.json"
    if not receipt_file.exists():
        raise ValueError(f"{previous} has not finished")
    receipt = json.loads(receipt_file.read_text())
    if receipt["stage"] != expected_stage:
        raise ValueError(f"expected a stage-{expected_stage} run, found stage {receipt['stage']}")
    checkpoint = previous / receipt["checkpoint"]
    if file_sha256(checkpoint) != receipt["checkpoint_sha256"]:
        raise ValueError("the earlier stage's checkpoint differs from its receipt")
    state = torch.load(checkpoint, map_location="cpu", weights_only=False)
    return {"stage": expected_stage, "fingerprint": receipt["fingerprint"], "checkpoint_sha256": receipt["checkpoint_sha256"]}, state


# ---- stage 1 -------------------------------------------------------------------------------------------------------------
def run_stage1(bundle: Bundle, batches: Callable[[int], torch.Tensor], cfg: Stage1Config, output) -> dict:
    torch.manual_seed(cfg.seed)
    run = _StageRun(1, output, cfg, None)
    switches = {layer: bundle.make_switch(layer) for layer in sorted(bundle.teacher_mixers)}
    holder = nn.ModuleDict({str(k): v for k, v in switches.items()})
    opt = torch.optim.AdamW(holder.parameters(), lr=cfg.lr, betas=(0.9, 0.95))
    resumed = run.resume({"switches": holder}, opt)
    step = resumed["step"] if resumed else 0
    last = {}
    while step < cfg.steps:
        for g in opt.param_groups:
            g["lr"] = D.cosine_lr(step, cfg.steps, cfg.lr, cfg.warmup_fraction, cfg.final_lr_fraction)
        last = D.latent_match_step(bundle.teacher, bundle.teacher_mixers, switches, opt, batches(step), loss_kind=cfg.loss)
        step += 1
        run.log({"step": step, "loss": last["loss"], "per_layer": {str(k): v for k, v in last["per_layer"].items()}, "grad_norm": last["grad_norm"]})
        if cfg.save_every and step % cfg.save_every == 0 and step < cfg.steps:
            run.save(step, {"switches": holder}, opt, {})
    return run.finish(step, {"switches": holder}, opt, {"loss": last.get("loss"), "layers": sorted(switches)})


def _installed_student(bundle: Bundle, switch_state: dict, layers) -> dict[int, nn.Module]:
    switches = {}
    for layer in layers:
        sw = bundle.make_switch(layer)
        sw.load_state_dict({k.split(".", 1)[1]: v for k, v in switch_state.items() if k.split(".", 1)[0] == str(layer)})
        bundle.install(bundle.student, layer, sw)
        switches[layer] = sw
    return switches


def _set_token_lr(opt, tokens_done: int, total: int) -> float:
    scale = D.wsd_lr(max(tokens_done, 1), total, 1.0)
    for g in opt.param_groups:
        g["lr"] = g["base_lr"] * scale
    return scale


def _clip(student: nn.Module, max_norm: float) -> float:
    g = float(torch.nn.utils.clip_grad_norm_([p for p in student.parameters() if p.grad is not None], max_norm))
    if not math.isfinite(g):
        raise FloatingPointError("non-finite gradient")
    return g


@torch.no_grad()
def composed_nll_gap(bundle: Bundle, ids: torch.Tensor) -> dict:
    """Teacher-forced evaluation of the composed student: mean forward KL and the next-token NLL of both models."""
    t_logits = bundle.teacher_head(bundle.teacher.hidden(ids))[:, :-1].float()
    s_logits = bundle.student_head(bundle.student.hidden(ids))[:, :-1].float()
    labels = ids[:, 1:]
    nll = lambda lg: float(torch.nn.functional.cross_entropy(lg.flatten(0, 1), labels.flatten()))
    return {"forward_kl": float(D._kl_rows(t_logits.flatten(0, 1), s_logits.flatten(0, 1)).mean()), "teacher_nll": nll(t_logits), "student_nll": nll(s_logits)}


# ---- stage 2 -------------------------------------------------------------------------------------------------------------
def run_stage2(bundle: Bundle, batches: Callable[[int], torch.Tensor], cfg: Stage2Config, output, *, stage1_dir, eval_ids=None) -> dict:
    torch.manual_seed(cfg.seed)
    lineage, state1 = lineage_of(stage1_dir, 1)
    run = _StageRun(2, output, cfg, lineage)
    switches = _installed_student(bundle, state1["modules"]["switches"], state1["extra"]["layers"])
    opt = D.two_timescale_optimizer(bundle.student, switches, lr=cfg.lr, backbone_lr_ratio=cfg.backbone_lr_ratio)
    resumed = run.resume({"student": bundle.student}, opt)
    step, tokens = (resumed["step"], resumed["extra"]["tokens"]) if resumed else (0, 0)
    before = composed_nll_gap(bundle, eval_ids) if eval_ids is not None else None
    kl = None
    while tokens < cfg.total_tokens:
        ids = batches(step)
        mask = torch.ones_like(ids, dtype=torch.bool)
        mask[:, -1] = False
        lr_scale = _set_token_lr(opt, tokens, cfg.total_tokens)
        opt.zero_grad(set_to_none=True)
        kl = D.chunked_kl_step(bundle.teacher.hidden, bundle.student.hidden, bundle.teacher_head, bundle.student_head, ids, mask,
                               direction="forward", chunk_tokens=cfg.chunk_tokens)
        gnorm = _clip(bundle.student, cfg.clip_norm)
        opt.step()
        step, tokens = step + 1, tokens + int(mask.sum())
        run.log({"step": step, "tokens": tokens, "forward_kl": kl, "grad_norm": gnorm, "lr_scale": lr_scale})
        if cfg.save_every and step % cfg.save_every == 0 and tokens < cfg.total_tokens:
            run.save(step, {"student": bundle.student}, opt, {"tokens": tokens, "layers": sorted(switches)})
    after = composed_nll_gap(bundle, eval_ids) if eval_ids is not None else None
    return run.finish(step, {"student": bundle.student}, opt, {"tokens": tokens, "layers": sorted(switches), "forward_kl": kl,
                                                                "evaluation_before": before, "evaluation_after": after})


# ---- stage 3 -------------------------------------------------------------------------------------------------------------
def run_stage3(bundle: Bundle, prompts: Callable[[int], torch.Tensor], cfg: Stage3Config, output, *, stage2_dir,
               anchor_batches: Callable[[int], torch.Tensor] | None = None) -> dict:
    torch.manual_seed(cfg.seed)
    lineage, state2 = lineage_of(stage2_dir, 2)
    run = _StageRun(3, output, cfg, lineage)
    switches = {}
    for layer in state2["extra"]["layers"]:                      # same modules in place, then the stage-2 weights
        switches[layer] = bundle.make_switch(layer)
        bundle.install(bundle.student, layer, switches[layer])
    bundle.student.load_state_dict(state2["modules"]["student"])
    opt = D.two_timescale_optimizer(bundle.student, switches, lr=cfg.lr, backbone_lr_ratio=cfg.backbone_lr_ratio)
    curriculum = D.HorizonCurriculum(cfg.min_gen_tokens)
    rollout_gen = torch.Generator().manual_seed(cfg.seed + 1)
    resumed = run.resume({"student": bundle.student}, opt)
    step, tokens = 0, 0
    if resumed:
        step, tokens = resumed["step"], resumed["extra"]["tokens"]
        curriculum = D.HorizonCurriculum(**resumed["extra"]["curriculum"])
        rollout_gen.set_state(resumed["extra"]["rollout_rng"])
    if cfg.anchor_kl_weight > 0 and anchor_batches is None:
        raise ValueError("an anchor weight needs teacher-forced anchor batches")
    logits_fn = lambda ids: bundle.student_head(bundle.student.hidden(ids))
    rkl = None
    while tokens < cfg.total_tokens:
        was = bundle.student.training
        bundle.student.eval()
        ids, mask = D.rollout(logits_fn, prompts(step), curriculum.gen_tokens, temperature=cfg.temperature, generator=rollout_gen)
        bundle.student.train(was)
        lr_scale = _set_token_lr(opt, tokens, cfg.total_tokens)
        opt.zero_grad(set_to_none=True)
        rkl = D.chunked_kl_step(bundle.teacher.hidden, bundle.student.hidden, bundle.teacher_head, bundle.student_head, ids, mask,
                                direction="reverse", chunk_tokens=cfg.chunk_tokens)
        anchor = None
        if cfg.anchor_kl_weight > 0:
            a_ids = anchor_batches(step)
            a_mask = torch.ones_like(a_ids, dtype=torch.bool)
            a_mask[:, -1] = False
            anchor = D.chunked_kl_step(bundle.teacher.hidden, bundle.student.hidden, bundle.teacher_head, bundle.student_head, a_ids, a_mask,
                                       direction="forward", chunk_tokens=cfg.chunk_tokens, scale=cfg.anchor_kl_weight)
        gnorm = _clip(bundle.student, cfg.clip_norm)
        opt.step()
        step, tokens = step + 1, tokens + int(mask.sum())
        grew = curriculum.update(rkl, max_gen_tokens=cfg.max_gen_tokens, plateau_steps=cfg.plateau_steps)
        run.log({"step": step, "tokens": tokens, "reverse_kl": rkl, "anchor_forward_kl": anchor, "grad_norm": gnorm, "lr_scale": lr_scale,
                 "gen_tokens": curriculum.gen_tokens, "horizon_grew": grew})
        if cfg.save_every and step % cfg.save_every == 0 and tokens < cfg.total_tokens:
            run.save(step, {"student": bundle.student}, opt, {"tokens": tokens, "curriculum": asdict(curriculum),
                                                              "rollout_rng": rollout_gen.get_state(), "layers": sorted(switches)})
    return run.finish(step, {"student": bundle.student}, opt, {"tokens": tokens, "reverse_kl": rkl, "gen_tokens": curriculum.gen_tokens,
                                                                "curriculum_phase": curriculum.phase, "layers": sorted(switches)})
