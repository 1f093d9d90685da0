"""Supervised fine-tuning on chat transcripts, and the export that hands the result to RL with its lineage.

* ``render_chat``    - a transcript (list of {role, content}) becomes token ids plus a loss mask that covers only
                       the assistant's tokens (and the end-of-turn token that teaches stopping).
* ``pack_examples``  - transcripts are concatenated into fixed-length rows, never splitting one across rows;
                       padding positions carry label -1.
* ``sft_step``       - one optimizer step of masked next-token cross-entropy (token mean over supervised positions).
* ``finalize_export``- writes the HF-layout export (config.json, model.safetensors, EXPORT.json last) with the
                       lineage an RL recipe's ``parent_stage`` / ``parent_tokens`` checks read: parent checkpoint
                       digest, the stage ("adapter_sft", "full_sft" or "package_sft"), supervised token count and the
                       data manifest digest.
Takes the place of the reference's SFT bootstrap and export finalisation (src/archlab/training/bootstrap.py,
sft_export.py), which compose an external trainer; the training loop here is the framework's own.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch
import torch.nn.functional as F

from ..ckpt.formats import export_hf, state_sha256
from ..contracts.substrate import sha256_file

STAGES = ("adapter_sft", "full_sft", "package_sft")


def render_chat(tokenizer, messages: list[dict]) -> tuple[list[int], list[int]]:
    """-> (ids, mask) with mask 1 on tokens the model must learn to produce."""
    sp = tokenizer.special
    ids, mask = [sp["<|bos|>"]], [0]
    for m in messages:
        role, text = m["role"], m["content"]
        if role not in ("user", "assistant"):
            raise ValueError("roles are user and assistant")
        body = tokenizer.encode(text)
        start, end = sp[f"<|{role}_start|>"], sp[f"<|{role}_end|>"]
        learn = 1 if role == "assistant" else 0
        ids += [start] + body + [end]
        mask += [0] + [learn] * len(body) + [learn]
    return ids, mask


def pack_examples(examples: list[tuple[list[int], list[int]]], row_len: int, pad_id: int = 0):
    """-> (inputs [R, row_len], labels [R, row_len]) with labels -1 where nothing is supervised.  An example longer
    than a row is truncated; examples are never split across rows."""
    rows_x, rows_y, cur_x, cur_y = [], [], [], []

    def flush():
        if cur_x:
            pad = row_len - len(cur_x)
            rows_x.append(cur_x + [pad_id] * pad)
            rows_y.append(cur_y + [-1] * pad)

    for ids, mask in examples:
        ids, mask = ids[: row_len + 1], mask[: row_len + 1]
        x = ids[:-1]
        y = [t if m else -1 for t, m in zip(ids[1:], mask[1:])]
        if len(cur_x) + len(x) > row_len:
            flush()
            cur_x, cur_y = [], []
        cur_x, cur_y = cur_x + x, cur_y + y
    flush()
    return torch.tensor(rows_x, dtype=torch.long), torch.tensor(rows_y, dtype=torch.long)


def sft_step(model, optimizer, inputs: torch.Tensor, labels: torch.Tensor, *, max_grad_norm: float = 1.0) -> dict:
    logits = model(inputs)
    loss = F.cross_entropy(logits.float().flatten(0, 1), labels.flatten(), ignore_index=-1)
    optimizer.zero_grad(set_to_none=True)
    loss.backward()
    gnorm = torch.nn.utils.clip_grad_norm_([p for p in model.parameters() if p.grad is not None], max_grad_norm)
    if not torch.isfinite(loss) or not torch.isfinite(gnorm):
        raise FloatingPointError("non-finite SFT loss or gradient")
    optimizer.step()
    return {"loss": float(loss.detach()), "grad_norm": float(gnorm), "supervised_tokens": int(labels.ne(-1).sum())}


def finalize_export(out_dir, model, config: dict, *, stage: str, supervised_tokens: int, parent_state_sha256: str,
                    data_manifest: Path, tokenizer_sha256: str | None = None) -> dict:
    if stage not in STAGES:
        raise ValueError(f"stage must be one of {STAGES}")
    if supervised_tokens <= 0:
        raise ValueError("an SFT endpoint needs a positive supervised token count")
    lineage = {"parent_stage": stage, "parent_tokens": int(supervised_tokens), "parent_state_sha256": parent_state_sha256,
               "data_manifest_sha256": sha256_file(Path(data_manifest)), "tokenizer_sha256": tokenizer_sha256}
    receipt = export_hf(out_dir, model.state_dict(), config, export_format="archlab-sft-hf-v1", lineage=lineage)
    (Path(out_dir) / "LINEAGE.json").write_text(json.dumps(lineage, indent=2, sort_keys=True))
    return receipt


def read_lineage(export_dir) -> dict:
    """What an RL recipe needs from its parent export; refuses exports without a receipt."""
    d = Path(export_dir)
    receipt = json.loads((d / "EXPORT.json").read_text())
    lineage = receipt.get("lineage") or json.loads((d / "LINEAGE.json").read_text())
    if lineage.get("parent_stage") not in STAGES or not lineage.get("parent_tokens"):
        raise ValueError("export carries no SFT lineage")
    return lineage
