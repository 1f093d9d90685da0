"""Training the byte-pair tokenizer of a pipeline run: bounded text, a round-trip check, the bits-per-byte weights.

Documents are cropped to ``doc_cap`` characters and the stream stops after ``max_chars`` characters, so tokenizer
training costs the same whatever the corpus size.  The trained tokenizer must reproduce a fixed probe text (ASCII,
digits, contractions, punctuation, CJK, emoji) exactly.  Beside ``tokenizer.json`` the directory receives
``token_bytes.pt``: the UTF-8 length of every token, 0 for special tokens, which turns a token-level loss into bits per
byte (a number that does not depend on the vocabulary size).  Token-length statistics go to the run's report card.
(Reference: src/archlab/speedrun/tok_train.py:1-125.)
"""
from __future__ import annotations

import argparse
import time
from pathlib import Path
from typing import Iterable, Iterator

import torch

from .tokenizer import BPETokenizer

PROBE = "Hello world! This is a test.\nNumbers: 123, 4567, 89\nContractions: I'm, you're, it's\nSpecial chars: @#$%^&*()\nUnicode: 你好世界 \U0001f30d"


def bounded_texts(documents: Iterable[str], *, max_chars: int, doc_cap: int) -> Iterator[str]:
    seen = 0
    for doc in documents:
        doc = doc[:doc_cap]
        seen += len(doc)
        yield doc
        if seen > max_chars:
            return


def train_tokenizer(documents: Iterable[str], out_dir, *, vocab_size: int = 32768, max_chars: int = 2_000_000_000, doc_cap: int = 10_000,
                    report=None) -> dict:
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    t0 = time.time()
    tokenizer = BPETokenizer.train(bounded_texts(documents, max_chars=max_chars, doc_cap=doc_cap), vocab_size)
    seconds = time.time() - t0
    if tokenizer.decode(tokenizer.encode(PROBE)) != PROBE:
        raise RuntimeError("the trained tokenizer does not round-trip the probe text")
    tokenizer.save(out / "tokenizer.json")
    weights = torch.tensor(tokenizer.token_bytes(), dtype=torch.int32)
    torch.save(weights, out / "token_bytes.pt")
    real = weights[weights > 0].float()
    stats = {"vocab_size": tokenizer.vocab_size, "num_special_tokens": len(tokenizer.special), "train_time": seconds, "tokenizer_sha256": tokenizer.sha256(),
             "token_bytes_min": int(real.min()), "token_bytes_max": int(real.max()), "token_bytes_mean": float(real.mean()),
             "token_bytes_std": float(real.std()) if real.numel() > 1 else 0.0}
    if report is not None:
        report.log("Tokenizer training", [{"max_chars": max_chars, "doc_cap": doc_cap, "vocab_size": vocab_size}, stats])
    return stats


def _documents(path: Path) -> Iterator[str]:
    """One document per line of every ``*.txt`` / ``*.jsonl`` (field ``text``) file under ``path``."""
    import json

    for file in sorted(p for p in path.rglob("*") if p.suffix in (".txt", ".jsonl")):
        with file.open() as f:
            for line in f:
                line = line.rstrip("\n")
                if line:
                    yield json.loads(line)["text"] if file.suffix == ".jsonl" else line


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Train the run's BPE tokenizer")
    ap.add_argument("--data", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--max-chars", type=int, default=2_000_000_000)
    ap.add_argument("--doc-cap", type=int, default=10_000)
    ap.add_argument("--vocab-size", type=int, default=32768)
    ap.add_argument("--report-dir", default=None)
    a = ap.parse_args(argv)
    report = None
    if a.report_dir:
        from ..services.run_report import get_report

        report = get_report(a.report_dir)
    stats = train_tokenizer(_documents(Path(a.data)), a.output, vocab_size=a.vocab_size, max_chars=a.max_chars, doc_cap=a.doc_cap, report=report)
    print({k: stats[k] for k in ("vocab_size", "train_time", "token_bytes_mean")})
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
