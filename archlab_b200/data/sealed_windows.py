"""A sealed pilot of supervised windows over a tokenised corpus: the selection is frozen with hashes, batches carry
exact assistant masks with ONE label shift, and ranks that run out of windows get an all-ignored batch of the same
shape family so that collectives stay aligned.

``seal_pilot`` writes ``windows.jsonl`` (one window per line: part file, start, length, assistant label spans in window
coordinates, target count) and ``PILOT_READY.json`` (format, split, context, counts, SHA-256 of the window file and of
the source corpus' ``DATA_READY.json``).  ``SealedWindows`` refuses a pilot whose window file or source changed, whose
split is not the requested one, or whose supervised-token total differs from the requested budget.  Windows are
shuffled once with a fixed seed, so effort / tool strata mix at optimizer-step scale instead of arriving as long
homogeneous runs of one source part; selection and masks stay those of the sealed pilot.

``batch(i)`` -> (inputs [1, C], labels [1, C], supervised count).  ``labels[t] = tokens[t + 1]`` inside the assistant
spans and -100 elsewhere; the sequence is padded to a power of two of at least 128 (or to the full context with
``pad_to_full``), which bounds the number of distinct shapes a captured step has to handle.  The count is re-derived
from the labels and must equal the sealed target count.  (Reference: src/archlab/automodel/deepseek_v41_data.py:16-85.)
"""
from __future__ import annotations

import hashlib
import json
import random
from collections import OrderedDict
from pathlib import Path

import numpy as np
import torch

from ..contracts.substrate import atomic_write_json

FORMAT = "archlab-sealed-window-pilot-v1"
IGNORE = -100


def seal_pilot(out_dir, source, windows: list[dict], *, split: str, context: int) -> dict:
    out, source = Path(out_dir), Path(source).resolve(strict=True)
    out.mkdir(parents=True, exist_ok=False)
    for w in windows:
        if w["length"] + 1 < 2 or w["length"] > context or sum(b - a for a, b in w["assistant_label_spans"]) != w["targets"]:
            raise ValueError("a window's spans do not add up to its target count, or it exceeds the context")
    body = "".join(json.dumps(w, sort_keys=True) + "\n" for w in windows).encode()
    (out / "windows.jsonl").write_bytes(body)
    manifest = {"format": FORMAT, "split": split, "context": context, "windows": len(windows), "supervised_tokens": sum(w["targets"] for w in windows),
                "windows_sha256": hashlib.sha256(body).hexdigest(), "source": str(source),
                "source_ready_sha256": hashlib.sha256((source / "DATA_READY.json").read_bytes()).hexdigest()}
    atomic_write_json(out / "PILOT_READY.json", manifest)
    return manifest


class SealedWindows:
    def __init__(self, root, *, expected_split: str, expected_budget: int | None = None, order_seed: int = 2234, vocab_size: int | None = None,
                 open_parts: int = 4):
        self.root = Path(root).resolve(strict=True)
        self.manifest = json.loads((self.root / "PILOT_READY.json").read_text())
        if self.manifest.get("format") != FORMAT or self.manifest["split"] != expected_split:
            raise ValueError("wrong pilot format or split")
        raw = (self.root / "windows.jsonl").read_bytes()
        if hashlib.sha256(raw).hexdigest() != self.manifest["windows_sha256"]:
            raise ValueError("the pilot's windows changed after sealing")
        self.windows = [json.loads(line) for line in raw.splitlines()]
        random.Random(order_seed).shuffle(self.windows)
        self.context, self.vocab_size, self.open_parts = self.manifest["context"], vocab_size, open_parts
        self.source = Path(self.manifest["source"]).resolve(strict=True)
        if hashlib.sha256((self.source / "DATA_READY.json").read_bytes()).hexdigest() != self.manifest["source_ready_sha256"]:
            raise ValueError("the source corpus changed after the pilot was prepared")
        if len(self.windows) != self.manifest["windows"]:
            raise ValueError("pilot window count mismatch")
        total = sum(w["targets"] for w in self.windows)
        if total != self.manifest["supervised_tokens"] or (expected_budget is not None and total != expected_budget):
            raise ValueError("the pilot does not match the requested supervised-token budget")
        self._parts: OrderedDict = OrderedDict()

    def __len__(self) -> int:
        return len(self.windows)

    def _part(self, name: str) -> np.ndarray:
        path = (self.source / name).resolve()
        if self.source not in path.parents:
            raise ValueError("pilot data escapes the tokenised corpus")
        if path not in self._parts:
            self._parts[path] = np.memmap(path, dtype=np.int32, mode="r")
            while len(self._parts) > self.open_parts:
                self._parts.popitem(last=False)
        self._parts.move_to_end(path)
        return self._parts[path]

    @staticmethod
    def _padded(length: int, context: int, pad_to_full: bool) -> int:
        return context if pad_to_full else min(context, max(128, 1 << (length - 1).bit_length()))

    def batch(self, index: int, *, device="cpu", pad_to_full: bool = False):
        if index >= len(self):                                          # a rank past its last window still takes part in the step
            width = self.context if pad_to_full else min(self.context, 128)
            return (torch.zeros(1, width, dtype=torch.int64, device=device), torch.full((1, width), IGNORE, dtype=torch.int64, device=device), 0)
        if index < 0:
            raise ValueError("invalid pilot index")
        w = self.windows[index]
        length = w["length"]
        tokens = torch.from_numpy(np.asarray(self._part(w["part"])[w["start"]:w["start"] + length + 1], dtype=np.int64).copy())
        if tokens.numel() != length + 1 or bool((tokens < 0).any()) or (self.vocab_size is not None and bool((tokens >= self.vocab_size).any())):
            raise ValueError("invalid token window")
        width = self._padded(length, self.context, pad_to_full)
        inputs = torch.zeros(1, width, dtype=torch.int64)
        labels = torch.full((1, width), IGNORE, dtype=torch.int64)
        inputs[0, :length] = tokens[:-1]
        count = 0
        for lo, hi in w["assistant_label_spans"]:
            lo, hi = max(0, lo), min(length, hi)
            if lo < hi:
                labels[0, lo:hi] = tokens[lo + 1:hi + 1]
                count += hi - lo
        if count != int((labels != IGNORE).sum()) or count != w["targets"]:
            raise ValueError("assistant targets were lost or counted twice")
        return inputs.to(device), labels.to(device), count


# ---- selecting a pilot with an EXACT supervised-token budget -----------------------------------------------------------
def shifted_window_spans(spans: list, start: int, length: int, *, limit: int | None = None) -> list[list[int]]:
    """Assistant TOKEN spans of a document -> half-open LABEL spans of the input window ``[start, start + length)``.

    Label ``t`` of a window is token ``start + t + 1``; a token at document position p is therefore label ``p - start - 1``
    and is supervised by the window whose inputs cover ``p - 1``.  Consecutive windows overlap by that one boundary token,
    so no assistant token is lost or counted twice.  ``limit`` cuts the selection after that many targets (the last
    window of a pilot stops exactly on the budget)."""
    out, left, previous = [], limit, 0
    for lo, hi in spans:
        if type(lo) is not int or type(hi) is not int or lo < previous or hi <= lo:
            raise ValueError("assistant spans must be sorted, non-overlapping, non-empty ranges")
        previous = hi
        a, b = max(lo, start + 1), min(hi, start + length + 1)
        if a >= b:
            continue
        if left is not None:
            b = min(b, a + left)
            left -= b - a
        if b > a:
            out.append([a - start - 1, b - start - 1])
        if left == 0:
            break
    return out


def select_pilot_windows(documents: list[dict], *, target_tokens: int, context: int, seed: int = 1234) -> tuple[list[dict], dict]:
    """``documents``: ``{"part", "offset", "tokens", "assistant_token_spans", ...}`` (offset = position of the document's
    first token in its part file).  Documents are shuffled deterministically; each selected document's windows are taken
    in order (every window starts a fresh context); windows without any target are skipped and counted; the selection
    stops on EXACTLY ``target_tokens`` targets or raises if the corpus is too small.  Returns the windows in the form
    ``seal_pilot`` takes and a summary."""
    if type(target_tokens) is not int or target_tokens < 1 or type(context) is not int or context < 2:
        raise ValueError("a positive supervised budget and a context of at least 2 are required")
    order = list(documents)
    random.Random(seed).shuffle(order)
    windows, targets, used_documents, skipped, resets = [], 0, 0, 0, 0
    for doc in order:
        spans = doc["assistant_token_spans"]
        if any(hi > doc["tokens"] for _, hi in spans):
            raise ValueError("supervision outside the source document")
        used = False
        for start in range(0, doc["tokens"] - 1, context):
            length = min(context, doc["tokens"] - 1 - start)
            selected = shifted_window_spans(spans, start, length, limit=target_tokens - targets)
            count = sum(hi - lo for lo, hi in selected)
            if not count:
                skipped += 1
                continue
            windows.append({"part": doc["part"], "start": doc["offset"] + start, "length": length, "assistant_label_spans": selected, "targets": count,
                            "context_reset": start > 0, **{k: doc[k] for k in ("problem_sha256", "mode", "has_tools") if k in doc}})
            targets += count
            resets += int(start > 0)
            used_documents += int(not used)
            used = True
            if targets == target_tokens:
                break
        if targets == target_tokens:
            break
    if targets != target_tokens:
        raise ValueError(f"the corpus holds only {targets} supervised tokens; {target_tokens} were requested")
    return windows, {"supervised_tokens": targets, "windows": len(windows), "documents": used_documents, "zero_target_windows_skipped": skipped,
                     "context_resets": resets, "seed": seed, "context": context}
