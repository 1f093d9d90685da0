"""Byte-level BPE tokenizer: train, encode, decode, special tokens, save / load.

The speedrun pipeline needs a tokenizer that can be trained on the corpus at hand and whose identity
(merge table hash) goes into the dataset manifest.  The reference uses rustbpe for training and tiktoken
for inference (src/archlab/speedrun/tokenizer.py); no such packages are assumed here - the merge
loop is plain Python over pre-split words (GPT-4 style split pattern), which is fast enough for the
vocabulary sizes of the small-scale campaigns, and encoding caches per word.  When the ``tokenizers``
package is importable, ``load_hf`` wraps a ``tokenizer.json`` behind the same interface.
"""
from __future__ import annotations

import hashlib
import json
from collections import Counter
from pathlib import Path

import regex

SPLIT_PATTERN = r"""'(?i:[sdmt]|ll|ve|re)|[^\r\n\p{L}\p{N}]?+\p{L}+|\p{N}{1,2}| ?[^\s\p{L}\p{N}]++[\r\n]*|\s*[\r\n]|\s+(?!\S)|\s+"""
SPECIAL_TOKENS = ("<|bos|>", "<|user_start|>", "<|user_end|>", "<|assistant_start|>", "<|assistant_end|>",
                  "<|python_start|>", "<|python_end|>", "<|output_start|>", "<|output_end|>")


class BPETokenizer:
    def __init__(self, merges: list[tuple[int, int]], special_tokens: tuple[str, ...] = SPECIAL_TOKENS, pattern: str = SPLIT_PATTERN):
        self.merges = [tuple(m) for m in merges]
        self.rank = {m: i for i, m in enumerate(self.merges)}
        self.pattern = pattern
        self._split = regex.compile(pattern)
        self.vocab = {i: bytes([i]) for i in range(256)}
        for i, (a, b) in enumerate(self.merges):
            self.vocab[256 + i] = self.vocab[a] + self.vocab[b]
        base = 256 + len(self.merges)
        self.special = {t: base + i for i, t in enumerate(special_tokens)}
        self._special_inv = {v: k for k, v in self.special.items()}
        self._cache: dict[bytes, list[int]] = {}

    # -- training ------------------------------------------------------------------------------------
    @classmethod
    def train(cls, texts, vocab_size: int, special_tokens: tuple[str, ...] = SPECIAL_TOKENS, pattern: str = SPLIT_PATTERN):
        n_merges = vocab_size - 256 - len(special_tokens)
        if n_merges < 0:
            raise ValueError("vocabulary smaller than bytes + special tokens")
        split = regex.compile(pattern)
        words = Counter()
        for t in texts:
            words.update(w.encode("utf-8") for w in split.findall(t))
        seqs = [(list(w), c) for w, c in words.items()]
        merges = []
        for step in range(n_merges):
            pairs = Counter()
            for ids, c in seqs:
                for p in zip(ids, ids[1:]):
                    pairs[p] += c
            if not pairs:
                break
            best = max(pairs, key=lambda p: (pairs[p], -p[0], -p[1]))       # deterministic tie-break
            new = 256 + step
            merges.append(best)
            for ids, _ in seqs:
                i, out = 0, []
                while i < len(ids):
                    if i + 1 < len(ids) and (ids[i], ids[i + 1]) == best:
                        out.append(new)
                        i += 2
                    else:
                        out.append(ids[i])
                        i += 1
                ids[:] = out
        return cls(merges, special_tokens, pattern)

    # -- encode / decode -----------------------------------------------------------------------------
    def _encode_word(self, w: bytes) -> list[int]:
        got = self._cache.get(w)
        if got is not None:
            return got
        ids = list(w)
        while len(ids) > 1:
            best = min(zip(ids, ids[1:]), key=lambda p: self.rank.get(p, 1 << 60))
            if best not in self.rank:
                break
            new, i, out = 256 + self.rank[best], 0, []
            while i < len(ids):
                if i + 1 < len(ids) and (ids[i], ids[i + 1]) == best:
                    out.append(new)
                    i += 2
                else:
                    out.append(ids[i])
                    i += 1
            ids = out
        self._cache[w] = ids
        return ids

    def encode(self, text: str, *, prepend_bos: bool = False, allow_special: bool = False) -> list[int]:
        out = [self.special["<|bos|>"]] if prepend_bos and "<|bos|>" in self.special else []
        parts = [text]
        if allow_special and self.special:
            parts = regex.split("(" + "|".join(regex.escape(t) for t in self.special) + ")", text)
        for part in parts:
            if allow_special and part in self.special:
                out.append(self.special[part])
            else:
                for w in self._split.findall(part):
                    out.extend(self._encode_word(w.encode("utf-8")))
        return out

    def decode(self, ids) -> str:
        chunks = []
        for i in ids:
            chunks.append(self._special_inv[i].encode() if i in self._special_inv else self.vocab[i])
        return b"".join(chunks).decode("utf-8", errors="replace")

    @property
    def vocab_size(self) -> int:
        return 256 + len(self.merges) + len(self.special)

    def token_bytes(self) -> list[int]:
        """UTF-8 length of every token (0 for special tokens): the weights of the bits-per-byte metric."""
        return [len(self.vocab[i]) for i in range(256 + len(self.merges))] + [0] * len(self.special)

    # -- identity / persistence ----------------------------------------------------------------------
    def sha256(self) -> str:
        body = json.dumps({"merges": self.merges, "special": list(self.special), "pattern": self.pattern}, separators=(",", ":"))
        return hashlib.sha256(body.encode()).hexdigest()

    def save(self, path: Path) -> None:
        Path(path).write_text(json.dumps({"format": "archlab-bpe-v1", "merges": self.merges, "special": list(self.special),
                                          "pattern": self.pattern, "sha256": self.sha256()}))

    @classmethod
    def load(cls, path: Path) -> "BPETokenizer":
        d = json.loads(Path(path).read_text())
        if d.get("format") != "archlab-bpe-v1":
            raise ValueError("not a tokenizer file of this framework")
        tok = cls([tuple(m) for m in d["merges"]], tuple(d["special"]), d["pattern"])
        if tok.sha256() != d["sha256"]:
            raise ValueError("tokenizer file is corrupt")
        return tok


def load_hf(path: Path):
    """Wrap a Hugging Face ``tokenizer.json`` (needs the ``tokenizers`` package) behind encode / decode."""
    from tokenizers import Tokenizer

    tk = Tokenizer.from_file(str(path))

    class _HF:
        vocab_size = tk.get_vocab_size()

        def encode(self, text, **_):
            return tk.encode(text, add_special_tokens=False).ids

        def decode(self, ids):
            return tk.decode(list(ids), skip_special_tokens=False)

    return _HF()


def core_metric(task_accuracies: dict[str, float], random_baselines: dict[str, float]) -> float:
    """CORE: mean over tasks of the accuracy centred at the task's random baseline, (acc - base) / (1 - base)."""
    if set(task_accuracies) != set(random_baselines) or not task_accuracies:
        raise ValueError("every task needs an accuracy and a baseline")
    return sum((task_accuracies[t] - random_baselines[t]) / (1.0 - random_baselines[t]) for t in task_accuracies) / len(task_accuracies)
