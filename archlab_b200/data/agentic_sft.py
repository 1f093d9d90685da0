"""Supervised data from agent trajectories: only tokens the model itself generated are targets, and every row is proven
to be what the serving stack would have seen.

* ``normalize_tool_messages``: one declared tool (default ``bash``), structured arguments restricted to the runtime
  contract, at most one call per assistant turn, every observation answering a pending call, the episode ending with an
  idle assistant message; the system prompt is the deployed agent's, supplied by the caller.
* ``encode_assistant_targets``: renders the conversation with the caller's ``render(history) -> ids`` and checks that
  every assistant turn's history is a token PREFIX of the full rendering (a template that re-serialises history
  differently cannot reproduce sampled turns and is refused); the loss mask covers each assistant turn up to and
  including exactly one EOS.  Nothing is clipped.
* ``trajectory_row``: rows straight from recorded token ids (``.npz`` with prompt ids, response ids, response mask and
  generation spans); mask and spans must agree; tokens outside the student vocabulary or special to one tokenizer only
  are refused; over-long episodes raise ``OverflowError`` (rejected whole, never truncated).
* ``task_split``: all seeds of a task land in the same split.  ``tokenizer_compatibility``: teacher and student must
  share the token model; ids that only one of them defines are returned for exclusion.
* ``PreparedTrajectories``: validated rows -> tensors, or packed ``(inputs, labels)`` rows for ``train.sft``.
(Reference: src/archlab/data/agentic_sft.py:117-254, teacher_trajectories.py:23-80.)
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Callable

import numpy as np

from ..contracts.substrate import sha256_file


def text_content(content) -> str:
    if content is None:
        return ""
    if isinstance(content, str):
        return content
    if any(part.get("type") != "text" for part in content):
        raise ValueError("only text content is supported")
    return "".join(part["text"] for part in content)


def normalize_tool_messages(messages: list[dict], *, system: str, tool: str = "bash", required: str = "command",
                            optional: dict | None = None) -> list[dict]:
    """``optional``: name -> (type, low, high) bounds of further arguments (default: ``timeout`` in (0, 300])."""
    optional = {"timeout": (int, 0, 300)} if optional is None else optional
    out, pending, calls = [{"role": "system", "content": system}], set(), 0
    for m in messages:
        role = m["role"]
        if role == "system":
            continue
        if role not in ("user", "assistant", "tool"):
            raise ValueError(f"unsupported message role: {role}")
        item = {"role": role, "content": text_content(m.get("content"))}
        if role == "assistant":
            if pending:
                raise ValueError("an assistant turn precedes its tool observations")
            tool_calls = m.get("tool_calls") or []
            if len(tool_calls) > 1:
                raise ValueError("one tool call per assistant turn")
            for call in tool_calls:
                fn = call["function"]
                args = json.loads(fn["arguments"]) if isinstance(fn["arguments"], str) else fn["arguments"]
                if fn["name"] != tool:
                    raise ValueError(f"trajectory uses a tool other than {tool}")
                if not isinstance(args, dict) or not args.get(required) or set(args) - {required, *optional}:
                    raise ValueError("tool arguments differ from the runtime contract")
                for name, (kind, low, high) in optional.items():
                    if name in args and (type(args[name]) is not kind or not low < args[name] <= high):
                        raise ValueError(f"tool argument {name} is outside the runtime contract")
                if not call.get("id"):
                    raise ValueError("missing tool-call identity")
                item["tool_calls"] = [{"id": call["id"], "type": "function", "function": {"name": tool, "arguments": json.dumps(args, ensure_ascii=False)}}]
                pending.add(call["id"])
                calls += 1
        elif role == "tool":
            if m.get("tool_call_id") not in pending:
                raise ValueError("a tool observation has no matching call")
            item["tool_call_id"] = m["tool_call_id"]
            pending.discard(m["tool_call_id"])
        out.append(item)
    if pending or not calls or len(out) < 4 or out[1]["role"] != "user":
        raise ValueError("incomplete tool trajectory")
    if out[-1]["role"] != "assistant" or out[-1].get("tool_calls"):
        raise ValueError("a trajectory must finish with an idle assistant response")
    return out


def encode_assistant_targets(render: Callable[[list[dict]], list[int]], messages: list[dict], *, eos_token_id: int, max_length: int,
                             request_prefix: Callable[[list[dict]], list[int]] | None = None) -> dict:
    """``request_prefix(history)``: the ids the gateway sends when it asks for the next assistant turn (defaults to
    ``render(history)``; differs when the template adds a generation prompt)."""
    request_prefix = request_prefix or render
    ids = render(messages)
    if len(ids) > max_length:
        raise ValueError(f"trajectory exceeds the context: {len(ids)} > {max_length}")
    mask, turns = [0] * len(ids), 0
    for i, m in enumerate(messages):
        if m["role"] != "assistant":
            continue
        before, after = request_prefix(messages[:i]), render(messages[:i + 1])
        if after[:len(before)] != before or ids[:len(after)] != after:
            raise ValueError("assistant history is not prefix-stable under this template")
        ends = [j for j in range(len(before), len(after)) if after[j] == eos_token_id]
        if len(ends) != 1 or ends[0] == len(before):
            raise ValueError("an assistant turn must contain content and exactly one EOS")
        mask[len(before):ends[0] + 1] = [1] * (ends[0] + 1 - len(before))
        turns += 1
    if not turns or mask[0] or not any(mask):
        raise ValueError("missing assistant targets")
    return {"input_ids": ids, "attention_mask": [1] * len(ids), "loss_mask": mask, "position_ids": list(range(len(ids)))}


def task_split(task: str, seed: int = 42, validation_fraction: float = 0.1) -> str:
    if not 0 < validation_fraction < 1:
        raise ValueError("validation_fraction must be between zero and one")
    bucket = int(hashlib.sha256(f"{seed}:{task}".encode()).hexdigest(), 16) / 2 ** 256
    return "validation" if bucket < validation_fraction else "train"


def tokenizer_compatibility(teacher, student) -> dict:
    a, b = (json.loads((Path(p) / "tokenizer.json").read_text()) for p in (teacher, student))
    for key in ("model", "normalizer", "pre_tokenizer", "post_processor", "decoder"):
        if a.get(key) != b.get(key):
            raise ValueError(f"teacher / student tokenizer mismatch: {key}")
    added = [{t["id"]: t for t in doc.get("added_tokens", [])} for doc in (a, b)]
    if any(added[0][k] != added[1][k] for k in added[0].keys() & added[1].keys()):
        raise ValueError("teacher / student tokenizer mismatch: shared added tokens")
    names = ("tokenizer.json", "tokenizer_config.json", "chat_template.jinja")
    return {"excluded_token_ids": sorted(added[0].keys() ^ added[1].keys()),
            "files": {label: {n: sha256_file(Path(root) / n) for n in names if (Path(root) / n).exists()} for label, root in (("teacher", teacher), ("student", student))}}


def trajectory_row(path, *, max_length: int, vocab_size: int, excluded_token_ids=(), prefix: str = "traj0_") -> dict:
    with np.load(path, allow_pickle=False) as data:
        prompt, response, mask, spans = (data[prefix + k] for k in ("prompt_ids", "response_ids", "response_mask", "generation_spans"))
    if any(x.ndim != 1 or x.dtype.kind not in "iu" for x in (prompt, response, mask)):
        raise ValueError("expected one-dimensional integer trajectory arrays")
    if not len(prompt) or len(response) != len(mask) or not np.isin(mask, (0, 1)).all() or not mask.any():
        raise ValueError("invalid trajectory mask")
    ids = np.concatenate((prompt, response)).astype(np.int64)
    if ids.min() < 0 or ids.max() >= vocab_size:
        raise ValueError("token outside the student vocabulary")
    if len(excluded_token_ids) and np.isin(ids, list(excluded_token_ids)).any():
        raise ValueError("trajectory contains a token that the two tokenizers do not share")
    if len(ids) > max_length:
        raise OverflowError(f"complete trajectory exceeds {max_length}: {len(ids)}")
    if spans.ndim != 2 or spans.shape[1] != 2 or spans.dtype.kind not in "iu":
        raise ValueError("invalid generation spans")
    expected, last = np.zeros(len(response), dtype=mask.dtype), 0
    for start, end in spans.tolist():
        if not last <= start <= end <= len(response):
            raise ValueError("overlapping or invalid generation spans")
        expected[start:end] = 1
        last = end
    if not np.array_equal(mask, expected):
        raise ValueError("generated-token mask and generation spans disagree")
    loss = np.concatenate((np.zeros(len(prompt), dtype=np.int64), mask.astype(np.int64)))
    return {"input_ids": ids.tolist(), "attention_mask": [1] * len(ids), "loss_mask": loss.tolist(), "position_ids": list(range(len(ids)))}


class PreparedTrajectories:
    """Validated pretokenised rows (a list, a ``.jsonl`` or a ``.parquet`` file)."""

    def __init__(self, rows, *, max_length: int = 131_072, eos_token_id: int | None = None, require_supervised_eos: bool = True, max_samples: int = -1):
        if isinstance(rows, (str, Path)):
            path = Path(rows)
            if path.suffix == ".parquet":
                import pyarrow.parquet as pq

                rows = pq.read_table(path).to_pylist()
            else:
                rows = [json.loads(line) for line in path.read_text().splitlines() if line.strip()]
        self.rows = list(rows)[:max_samples] if max_samples > 0 else list(rows)
        for r in self.rows:
            ids, mask = r["input_ids"], r["loss_mask"]
            if not ids or len(ids) > max_length or len(ids) != len(mask) or mask[0] != 0 or not any(mask) or set(mask) - {0, 1}:
                raise ValueError("invalid prepared token / mask contract")
            if require_supervised_eos and eos_token_id is not None and not any(t == eos_token_id and m for t, m in zip(ids, mask)):
                raise ValueError("prepared trajectory has no supervised EOS")
            if r.get("attention_mask", [1] * len(ids)) != [1] * len(ids):
                raise ValueError("prepared trajectory contains padding")
            if r.get("position_ids", list(range(len(ids)))) != list(range(len(ids))):
                raise ValueError("prepared position ids must be contiguous")

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        import torch

        r = self.rows[i]
        n = len(r["input_ids"])
        return {"input_ids": torch.tensor(r["input_ids"]), "attention_mask": torch.ones(n, dtype=torch.long),
                "loss_mask": torch.tensor(r["loss_mask"]), "position_ids": torch.arange(n)}

    def examples(self) -> list[tuple[list[int], list[int]]]:
        """(ids, mask) per row, the form ``train.sft.pack_examples`` takes."""
        return [(r["input_ids"], r["loss_mask"]) for r in self.rows]

    def supervised_tokens(self) -> int:
        return sum(sum(r["loss_mask"]) for r in self.rows)
