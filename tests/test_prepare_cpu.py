import json

import pytest

from archlab_b200.data import prepare as P
from archlab_b200.data.tokenizer import BPETokenizer


def test_token_parts_round_trip_and_tamper_detection(tmp_path):
    docs = ["alpha beta gamma " * 5, "delta epsilon", "zeta " * 30]
    tok = BPETokenizer.train(docs, 256 + 9 + 12)
    eod = tok.special["<|bos|>"]
    m = P.prepare_token_parts(docs, tok, tmp_path / "ds", part_tokens=50, eod=eod)
    assert m["documents"] == 3 and sum(p["tokens"] for p in m["parts"]) == m["tokens"] and all(p["tokens"] <= 50 for p in m["parts"])
    assert P.verify_token_parts(tmp_path / "ds")["tokenizer_sha256"] == tok.sha256()
    stream = [int(t) for i in range(len(m["parts"])) for t in P.read_part(tmp_path / "ds", i)]
    want = []
    for d in docs:
        want += tok.encode(d) + [eod]
    assert stream == want
    with pytest.raises(FileExistsError):
        P.prepare_token_parts(docs, tok, tmp_path / "ds", part_tokens=50, eod=eod)
    part = tmp_path / "ds" / m["parts"][0]["file"]
    data = bytearray(part.read_bytes())
    data[0] ^= 1
    part.write_bytes(bytes(data))
    with pytest.raises(ValueError):
        P.verify_token_parts(tmp_path / "ds")


def test_math_filter_and_group_split():
    recs = [{"problem": "What is 1+1?", "answer": "2"}, {"problem": "what  is 1+1?", "answer": "2.0"}, {"problem": "", "answer": "3"},
            {"problem": "x?", "answer": None}, {"problem": "Half of one?", "answer": "\\frac{1}{2}", "source": "s"}]
    kept, stats = P.filter_math_records(recs)
    assert stats == {"read": 5, "invalid": 2, "duplicate": 1, "kept": 2} and kept[1]["source"] == "s"
    sides = [P.split_by_group(f"g{i}", 7, 0.25) for i in range(400)]
    assert 60 < sum(sides) < 140 and sides == [P.split_by_group(f"g{i}", 7, 0.25) for i in range(400)]
