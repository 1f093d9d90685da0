"""Evaluation of a base-model checkpoint in three independent modes: ``core`` (the multiple-choice task suite with centred
accuracies), ``bpb`` (bits per byte on token batches, vocabulary-size invariant) and ``sample`` (greedy continuations of
a prompt set).  One entry point, one result file, one report-card section.

``evaluate_checkpoint`` takes the model and whatever each selected mode needs (a task bundle, batches plus the
tokenizer's ``token_bytes`` weights, prompts) and returns ``{"core": ..., "bpb": {split: value}, "samples": [...]}`` with
only the selected keys; an unknown mode or a selected mode without its inputs is an error rather than a silent skip.
The command line loads a speedrun bundle (``ckpt.speedrun.build_model``), the run's tokenizer and token parts, and
writes ``base_eval_<step>.json`` (rank 0).  (Reference: src/archlab/speedrun/base_eval.py:121-374.)
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path
from typing import Iterable

import torch

from .evaluation import evaluate_bpb, evaluate_core, generate_batch, load_prompts, load_task_bundle

MODES = ("core", "bpb", "sample")


def parse_modes(text: str) -> set[str]:
    modes = {m.strip() for m in text.split(",") if m.strip()}
    bad = modes - set(MODES)
    if bad or not modes:
        raise ValueError(f"invalid evaluation modes {sorted(bad)}; valid: {MODES}")
    return modes


def evaluate_checkpoint(model, modes: set[str], *, tasks: dict | None = None, max_per_task: int = -1, bpb_batches: dict[str, Iterable] | None = None,
                        token_bytes: torch.Tensor | None = None, prompts: list[list[int]] | None = None, sample_tokens: int = 16, decode=None,
                        rank: int = 0, world: int = 1, core_encode=None, core_max_tokens: int | None = None) -> dict:
    out: dict = {}
    if "core" in modes:
        if tasks is None:
            raise ValueError("core evaluation needs a task bundle")
        if isinstance(tasks, list):                                            # the published directory layout, all three task types
            from ..evaluation.core_tasks import evaluate_bundle

            device, was_training = next(model.parameters()).device, model.training
            model.eval()
            out["core"] = evaluate_bundle(lambda ids: model(ids), core_encode, tasks, max_per_task=max_per_task, rank=rank, world=world,
                                          device=device, max_tokens=core_max_tokens)
            model.train(was_training)
        else:
            out["core"] = evaluate_core(model, tasks, max_per_task=max_per_task, rank=rank, world=world)
    if "bpb" in modes:
        if not bpb_batches or token_bytes is None:
            raise ValueError("bpb evaluation needs batches per split and the tokenizer's token_bytes")
        out["bpb"] = {split: evaluate_bpb(model, batches, token_bytes) for split, batches in bpb_batches.items()}
    if "sample" in modes:
        if not prompts:
            raise ValueError("sampling needs prompts")
        if rank == 0:
            generated = generate_batch(model, prompts, sample_tokens, temperature=0.0)
            out["samples"] = [{"prompt": p, "tokens": g, **({"text": decode(p + g)} if decode else {})} for p, g in zip(prompts, generated)]
    return out


def part_batches(part: torch.Tensor, batch_size: int, seq_len: int, tokens: int, device):
    """Consecutive (inputs, targets) batches over the first ``tokens`` tokens of a flat token tensor."""
    per = batch_size * seq_len
    for start in range(0, min(tokens, part.numel() - 1) - per + 1, per):
        block = part[start:start + per + 1].to(device=device, dtype=torch.long)
        yield block[:-1].view(batch_size, seq_len), block[1:].view(batch_size, seq_len)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Base-model evaluation: core, bpb, sample")
    ap.add_argument("--checkpoint-dir", required=True)
    ap.add_argument("--step", type=int, default=None, help="default: the last step in the directory")
    ap.add_argument("--eval", default="core,bpb,sample")
    ap.add_argument("--tokenizer", required=True, help="directory with tokenizer.json and token_bytes.pt")
    ap.add_argument("--task-bundle", default=None)
    ap.add_argument("--max-per-task", type=int, default=-1)
    ap.add_argument("--data", default=None, help="token-part dataset (DATA_READY.json) for bpb")
    ap.add_argument("--device-batch-size", type=int, default=32)
    ap.add_argument("--split-tokens", type=int, default=40 * 524288)
    ap.add_argument("--prompt-file", default=None)
    ap.add_argument("--report-dir", default=None)
    a = ap.parse_args(argv)
    from ..ckpt.speedrun import build_model, find_last_step
    from ..data.prepare import read_part
    from ..data.tokenizer import BPETokenizer

    modes = parse_modes(a.eval)
    device = "cuda" if torch.cuda.is_available() else "cpu"
    step = a.step if a.step is not None else find_last_step(a.checkpoint_dir)
    model, meta = build_model(a.checkpoint_dir, step, device, phase="eval")
    tokenizer = BPETokenizer.load(Path(a.tokenizer) / "tokenizer.json")
    seq_len = meta["model_config"]["sequence_len"]
    kwargs: dict = {"decode": tokenizer.decode}
    if "core" in modes:
        if Path(a.task_bundle).is_dir():
            from ..evaluation.core_tasks import read_bundle

            kwargs.update(tasks=read_bundle(a.task_bundle), max_per_task=a.max_per_task, core_max_tokens=seq_len,
                          core_encode=lambda text: tokenizer.encode(text, prepend_bos=True))
        else:
            kwargs.update(tasks=load_task_bundle(a.task_bundle, tokenizer), max_per_task=a.max_per_task)
    if "bpb" in modes:
        part = torch.from_numpy(read_part(Path(a.data), 0).astype("int64"))
        kwargs.update(token_bytes=torch.load(Path(a.tokenizer) / "token_bytes.pt").to(device),
                      bpb_batches={"val": part_batches(part, a.device_batch_size, seq_len, a.split_tokens, device)})
    if "sample" in modes:
        kwargs.update(prompts=load_prompts(a.prompt_file, tokenizer))
    result = {"step": step, "modes": sorted(modes), **evaluate_checkpoint(model, modes, **kwargs)}
    out = Path(a.checkpoint_dir) / f"base_eval_{step:06d}.json"
    out.write_text(json.dumps(result, indent=1, default=str) + "\n")
    if a.report_dir:
        from ..services.run_report import get_report

        section = [{"step": step}]
        if "core" in result:
            section.append({"CORE": result["core"]["core_metric"], **result["core"]["centered_results"]})
        if "bpb" in result:
            section.append({f"{k} bpb": v for k, v in result["bpb"].items()})
        get_report(a.report_dir).log("Base model evaluation", section)
    print(json.dumps({k: v for k, v in result.items() if k != "samples"}, default=str))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
