"""Rendering reasoning-chat corpora with a model's OWN encoder and supervising exactly the assistant's characters.

The encoder is not re-implemented: ``load_pinned_encoder`` imports the model publisher's encoding file only if its
SHA-256 equals the reviewed one.  Around it:

* ``coalesce_reasoning_fragments``: some corpora split one assistant turn into several messages (reasoning-only
  fragments followed by the answer or call).  Fragments that carry ONLY reasoning are joined into the final message with
  a documented separator, every character kept; anything else (two complete answers in a row, a fragment with a tool
  call) is left as separate native messages.  Each repair is recorded with source indices and hashes.
* ``render_conversation``: the full text, and for every assistant message the character span it adds, proven by
  prefix-stability: text(messages[:i]) and text(messages[:i+1]) must both be prefixes of the full text.  Conversations
  that end with a tool call or a non-assistant message are kept and flagged, nothing is fabricated.
* ``token_spans``: character spans -> token index ranges from the tokenizer's offsets; a token that straddles a
  supervision boundary is an error (a merge across the boundary would leak prompt characters into the target).
(Reference: src/archlab/preprocessing/deepseek_v41.py:21-180.)
"""
from __future__ import annotations

import copy
import hashlib
import importlib.util
from bisect import bisect_left
from pathlib import Path
from typing import Callable

SEPARATOR = "\n\n"
_FRAGMENT_KEYS = {"role", "content", "reasoning_content", "tool_calls"}


def load_pinned_encoder(path, sha256: str, module_name: str = "archlab_pinned_chat_encoder"):
    path = Path(path)
    if hashlib.sha256(path.read_bytes()).hexdigest() != sha256:
        raise ValueError("the encoder file is not the reviewed revision")
    spec = importlib.util.spec_from_file_location(module_name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def _reasoning_only(m: dict) -> bool:
    return not m.get("content") and not m.get("tool_calls") and isinstance(m.get("reasoning_content"), str) and bool(m["reasoning_content"])


def coalesce_reasoning_fragments(messages: list[dict]) -> tuple[list[dict], list[dict]]:
    out, repairs, i = [], [], 0
    while i < len(messages):
        j = i + 1
        if messages[i].get("role") == "assistant":
            while j < len(messages) and messages[j].get("role") == "assistant":
                j += 1
        group = messages[i:j]
        if len(group) == 1:
            out.append(group[0])
        elif not all(_reasoning_only(m) for m in group[:-1]):
            out.extend(group)
            repairs.append({"policy": "keep-consecutive-assistants", "source_message_indices": list(range(i, j)), "messages_merged": False})
        else:
            for m in group[:-1]:
                extra = [k for k, v in m.items() if k not in _FRAGMENT_KEYS and v not in (None, "", [], {})]
                if extra:
                    raise ValueError(f"cannot discard assistant fragment field {extra[0]!r}")
            parts = [m.get("reasoning_content") or "" for m in group]
            if any(not isinstance(p, str) for p in parts):
                raise ValueError("assistant reasoning must be text")
            final = copy.deepcopy(group[-1])
            final["reasoning_content"] = SEPARATOR.join(parts)
            out.append(final)
            repairs.append({"policy": "merge-reasoning-only-prefixes", "source_message_indices": list(range(i, j)), "separator": SEPARATOR,
                            "reasoning_character_lengths": [len(p) for p in parts],
                            "reasoning_sha256": [hashlib.sha256(p.encode()).hexdigest() for p in parts]})
        i = j
    return out, repairs


def check_messages(messages: list[dict], tools: list | None = None) -> list[dict]:
    """Text-only messages of the four roles; tool definitions travel on the (possibly added, empty) system message."""
    messages = copy.deepcopy(messages)
    for m in messages:
        if m.get("role") not in ("system", "user", "assistant", "tool"):
            raise ValueError("unsupported source message role")
        if not isinstance(m.get("content", ""), str):
            raise ValueError("this corpus contract is text-only")
    if tools:
        if messages[0]["role"] != "system":
            messages.insert(0, {"role": "system", "content": ""})
        if messages[0].get("tools") and messages[0]["tools"] != tools:
            raise ValueError("conflicting source tool definitions")
        messages[0]["tools"] = copy.deepcopy(tools)
    return messages


def render_conversation(encode: Callable[[list[dict]], str], messages: list[dict], *, tools: list | None = None, bos: str | None = None,
                        eos: str | None = None) -> tuple[str, list[dict], dict]:
    last = len(messages) - 1
    merged, repairs = coalesce_reasoning_fragments(messages)
    merged = check_messages(merged, tools)
    if merged[-1].get("tool_calls"):
        repairs.append({"policy": "keep-terminal-tool-call", "source_message_indices": [last], "complete_answer": False})
    if merged[-1]["role"] != "assistant":
        repairs.append({"policy": "keep-non-assistant-ending", "source_message_indices": [last], "terminal_role": merged[-1]["role"], "complete_answer": False})
    text = encode(merged)
    if bos is not None and not text.startswith(bos):
        raise ValueError("the encoding lost the conversation start")
    if eos is not None and merged[-1]["role"] == "assistant" and not text.endswith(eos):
        raise ValueError("the encoding lost the assistant ending")
    spans = []
    for i, m in enumerate(merged):
        if m["role"] != "assistant":
            continue
        if i == 0:
            raise ValueError("an assistant-only source needs an explicit policy")
        before, through = encode(merged[:i]), encode(merged[:i + 1])
        if not text.startswith(before) or not text.startswith(through):
            raise ValueError("the encoding is not prefix-stable at assistant boundaries")
        if len(before) >= len(through):
            raise ValueError("empty assistant supervision span")
        spans.append((len(before), len(through)))
    meta = {"assistant_character_spans": spans}
    if repairs:
        meta["message_repairs"] = repairs
    return text, merged, meta


def token_spans(offsets: list[tuple[int, int]], character_spans: list[tuple[int, int]]) -> list[list[int]]:
    """Token index ranges [begin, stop) of the targets, BEFORE the next-token shift (the trainer shifts once)."""
    starts, ends = [a for a, _ in offsets], [b for _, b in offsets]
    out = []
    for left, right in character_spans:
        begin, stop = bisect_left(starts, left), bisect_left(starts, right)
        if begin == stop or starts[begin] != left or ends[stop - 1] != right:
            raise ValueError("the tokenizer crosses an assistant supervision boundary")
        if begin and ends[begin - 1] > left:
            raise ValueError("a token overlaps an assistant supervision boundary")
        out.append([begin, stop])
    return out
