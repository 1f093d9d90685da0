"""Benchmark overlap audit against an RL problem set and a prepared corpus."""
import json

import pytest

from archlab_b200.data import prepare_job as pj
from archlab_b200.data.rl_problems import Exposure, problem_key, select_problems, write_problem_set
from archlab_b200.evaluation import overlap_audit as oa

CASES = [{"id": "bench-1", "question": "Find  x  if \\left( x-3 \\right)^2 = 0."}, {"id": "bench-2", "question": "What is 2+2?"},
         {"id": "bench-3", "question": "What is -3 + 5?"}]


def test_normalisation_keeps_signs():
    assert oa.normalized_text("Find x if \\left( x − 3 \\right)^2 = 0.") == oa.normalized_text(CASES[0]["question"]) == "findxifx-320"
    assert oa.normalized_text("What is -3 + 5?") != oa.normalized_text("What is 3 + 5?")


def test_rl_problem_sets_are_checked_by_hash_and_by_contained_text(tmp_path):
    rows = [{"problem": "Find x if \\left( x-3 \\right)^2 = 0.", "expected_answer": "3", "uuid": "u1"},                # exact (whitespace-normalised)
            {"problem": "Warm-up. WHAT IS 2 + 2 ? Explain.", "expected_answer": "4", "uuid": "u2"},                    # contained after normalisation
            {"problem": "What is 3 + 5?", "expected_answer": "8", "uuid": "u3"}] + [
            {"problem": f"Compute {i} + 1.", "expected_answer": str(i + 1), "uuid": f"f{i}"} for i in range(6)]
    train, held, counts = select_problems(rows, Exposure(), train_size=6, heldout_size=3, seed=1, canonicalizer=lambda s: s.strip())
    write_problem_set(tmp_path / "rl", train, held, counts, Exposure(), seed=1)
    report = oa.audit_rl(CASES, tmp_path / "rl")
    found = {(m["problem_id"], m["method"].split()[0]) for m in report["matches"]}
    assert found == {("bench-1", "exact"), ("bench-2", "format-normalised")} and sum(report["rows"].values()) == 9
    with (tmp_path / "rl" / "train.jsonl").open("a") as f:
        f.write("{}\n")
    with pytest.raises(ValueError, match="changed after it was sealed"):
        oa.audit_rl(CASES, tmp_path / "rl")


class Tok:
    def encode(self, text):
        return [ord(c) % 50 for c in text]


def test_prepared_corpora_report_what_the_cursor_had_read(tmp_path):
    problems = ["Compute 1 + 1.", CASES[1]["question"], "Compute 7 * 6.", CASES[2]["question"]]
    rows = [{"id": f"r{i}", "problem": p} for i, p in enumerate(problems)]
    tasks = [{"id": "t0", "source": "s", "row_start": 0, "rows": 2}, {"id": "t1", "source": "s", "row_start": 2, "rows": 2}]
    pj.Contract.create(tmp_path / "corpus", tokenizer_sha256="t" * 64, renderer_sha256="r" * 64, tasks=tasks)
    for t in tasks:
        pj.run_task(tmp_path / "corpus", t["id"], rows[t["row_start"]:t["row_start"] + 2], lambda r: r["problem"], Tok(), eod=0,
                    meta_of=lambda r: {"problem_sha256": problem_key(r["problem"])})
    first_doc = len(problems[0]) + 1
    early = oa.audit_prepared(CASES, tmp_path / "corpus", tokens_read=first_doc + 1, context=4, global_windows_per_step=2)
    assert [e["problem_id"] for e in early["retained_document_matches"]] == ["bench-2", "bench-3"]
    assert early["seen_problem_ids"] == ["bench-2"] and early["cursor_tokens"] % 8 == 0 and early["cursor_tokens"] >= first_doc + 1
    late = oa.audit_prepared(CASES, tmp_path / "corpus", tokens_read=10_000, context=4, global_windows_per_step=2)
    assert late["seen_problem_ids"] == ["bench-2", "bench-3"] and late["documents_scanned"] == 4
    (tmp_path / "cases.jsonl").write_text("".join(json.dumps(c) + "\n" for c in CASES))
    full = oa.audit(tmp_path / "cases.jsonl", prepared=tmp_path / "corpus", tokens_read=10_000, context=4, global_windows_per_step=2)
    assert full["cases"] == 3 and "paraphrases" in full["limitation"] and "rl" not in full
    sidecar = next((tmp_path / "corpus" / "parts" / "t0").glob("*train.metadata.jsonl.gz"))
    sidecar.write_bytes(sidecar.read_bytes() + b"x")
    with pytest.raises(ValueError, match="sealed document metadata changed"):
        oa.audit_prepared(CASES, tmp_path / "corpus", tokens_read=100, context=4, global_windows_per_step=2)
