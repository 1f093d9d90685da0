"""Tokenizer training job: bounded text, probe round trip, bits-per-byte weights, report section."""
import json

import torch

from archlab_b200.data.tok_train import PROBE, bounded_texts, main, train_tokenizer
from archlab_b200.data.tokenizer import BPETokenizer
from archlab_b200.services.run_report import RunReport


def test_text_is_bounded():
    docs = ["a" * 50, "b" * 5, "c" * 50, "d" * 50]
    got = list(bounded_texts(docs, max_chars=25, doc_cap=10))
    assert got == ["a" * 10, "b" * 5, "c" * 10, "d" * 10][:4] and sum(map(len, got[:3])) == 25     # stops after the limit is exceeded
    assert list(bounded_texts(docs, max_chars=12, doc_cap=10)) == ["a" * 10, "b" * 5]


def test_job_writes_tokenizer_weights_and_report(tmp_path):
    docs = ["the quick brown fox jumps over the lazy dog " * 20, "hello hello world world " * 30, PROBE] * 3
    report = RunReport(tmp_path / "report")
    report.reset({"commit": "x"})
    stats = train_tokenizer(docs, tmp_path / "tok", vocab_size=300, report=report)
    tok = BPETokenizer.load(tmp_path / "tok" / "tokenizer.json")
    weights = torch.load(tmp_path / "tok" / "token_bytes.pt")
    assert stats["vocab_size"] == tok.vocab_size == weights.numel() and stats["tokenizer_sha256"] == tok.sha256()
    assert int((weights == 0).sum()) == stats["num_special_tokens"] and stats["token_bytes_max"] >= 2 and stats["token_bytes_min"] == 1
    ids = tok.encode("the quick brown fox")
    assert int(weights[ids].sum()) == len("the quick brown fox".encode())                          # bytes are conserved by the weights
    section = json.loads((tmp_path / "report" / "tokenizer-training.json").read_text())
    assert section["fields"]["vocab_size"] == stats["vocab_size"] and "token_bytes_mean" in section["fields"]
    (tmp_path / "data").mkdir()
    (tmp_path / "data" / "a.txt").write_text("\n".join(docs[:2]) + "\n")
    (tmp_path / "data" / "b.jsonl").write_text(json.dumps({"text": PROBE}) + "\n")
    assert main(["--data", str(tmp_path / "data"), "--output", str(tmp_path / "tok2"), "--vocab-size", "280"]) == 0
    assert (tmp_path / "tok2" / "token_bytes.pt").exists()
