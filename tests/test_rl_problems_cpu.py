"""RL problem-set selection: exposure, poisoning by conflicting golds, aliasing, stable split."""
import gzip
import json

import pytest

from archlab_b200.data import rl_problems as rp
from archlab_b200.services.rewards import canonical_math_answer


def _rows(n=40):
    rows = []
    for i in range(n):
        rows.append({"problem": f"What is {i} + {i}?", "expected_answer": str(2 * i), "uuid": f"u{i}", "_source": {"file": "a.parquet", "row": i}})
    return rows


def test_selection_rules(tmp_path):
    rows = _rows()
    rows.append({"problem": "What  is 3 +   3?", "expected_answer": "6", "uuid": "u3", "_source": {"file": "a.parquet", "row": 100}})     # duplicate text
    rows.append({"problem": "What is 4 + 4?", "expected_answer": "9", "uuid": "u4", "_source": {"file": "b.parquet", "row": 0}})          # conflicting gold
    rows.append({"problem": "What is 5 + 5?", "expected_answer": "ten-ish words", "uuid": "u5", "_source": {"file": "b.parquet", "row": 1}})  # unsupported gold
    rows.append({"problem": "A different text", "expected_answer": "1", "uuid": "u6", "_source": {"file": "b.parquet", "row": 2}})        # id u6 with two texts
    rows.append({"problem": "", "expected_answer": "1"})
    side = tmp_path / "sft.metadata.jsonl.gz"
    side.write_bytes(gzip.compress((json.dumps({"problem": "What is 7 + 7?"}) + "\n" + json.dumps({"uuid": "u8"}) + "\n").encode()))
    exposure = rp.Exposure().add_metadata(side)
    canon = lambda s: canonical_math_answer(s)
    train, held, counts = rp.select_problems(rows, exposure, train_size=20, heldout_size=5, seed=1, canonicalizer=canon)
    ids = {r["id"] for r in train} | {r["id"] for r in held}
    key = rp.problem_key
    assert len(train) == 20 and len(held) == 5 and not {r["id"] for r in train} & {r["id"] for r in held}
    for gone in ("What is 7 + 7?", "What is 8 + 8?", "What is 4 + 4?", "What is 5 + 5?", "What is 6 + 6?", "A different text"):
        assert key(gone) not in ids
    assert counts["previously_exposed_problem_or_id"] == 2 and counts["unsupported_gold"] == 1 and counts["invalid_or_long_problem"] == 1
    assert counts["conflicting_or_aliased_problems"] == 4 and counts["eligible_unique_problems"] == 35      # 38 unexposed + 1 new text - 4 dropped
    dup = next((r for r in train + held if r["id"] == key("What is 3 + 3?")), None)
    assert dup is None or dup["source"]["row"] == 3                      # the earliest source represents a duplicate
    # the choice is stable under appended rows and changes with the seed
    more = rows + [{"problem": f"Extra {i}", "expected_answer": "1", "uuid": f"x{i}", "_source": {"file": "z.parquet", "row": i}} for i in range(5)]
    _, held2, _ = rp.select_problems(more, exposure, train_size=20, heldout_size=5, seed=1, canonicalizer=canon)
    assert len({r["id"] for r in held} & {r["id"] for r in held2}) >= 3
    _, held3, _ = rp.select_problems(rows, exposure, train_size=20, heldout_size=5, seed=2, canonicalizer=canon)
    assert [r["id"] for r in held3] != [r["id"] for r in held]
    with pytest.raises(ValueError, match="eligible unique problems"):
        rp.select_problems(rows, exposure, train_size=100, heldout_size=5, seed=1, canonicalizer=canon)
    manifest = rp.write_problem_set(tmp_path / "set", train, held, counts, exposure, seed=1)
    assert manifest["files"]["train"]["records"] == 20 and manifest["exposure"]["artifacts"][0]["path"].endswith("sft.metadata.jsonl.gz")
    assert len((tmp_path / "set" / "heldout.jsonl").read_text().splitlines()) == 5


def test_problem_key_normalises_whitespace_and_unicode():
    assert rp.problem_key("a  b\n c") == rp.problem_key("a b c") and rp.problem_key("é") == rp.problem_key("é")
    with pytest.raises(ValueError):
        rp.problem_key("   ")
