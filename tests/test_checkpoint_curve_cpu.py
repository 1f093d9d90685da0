"""Choice benchmark over checkpoints: span encoding, order-preserving scoring, identity-bound caching, aggregation."""
import json

import pytest
import torch

from archlab_b200.evaluation import checkpoint_curve as cc


def encode(text):                       # byte tokenizer with a leading BOS (id 1)
    return [1] + [3 + b for b in text.encode()]


EXAMPLES = [{"goal": "open a jar", "choices": ["twist the lid", "eat it"], "label": 0},
            {"goal": "dry hands", "choices": ["use water", "use a towel"], "label": 1},
            {"goal": "light", "choices": ["switch on", "dig"], "label": 0}]


def favouring(text_bytes):
    """A 'model' whose next-token distribution likes the bytes of the given words."""
    liked = {3 + b for b in text_bytes}

    def logits(ids):
        out = torch.zeros(*ids.shape, 260)
        out[..., sorted(liked)] = 3.0
        return out
    return logits


def test_spans_are_what_the_choice_adds_to_the_context():
    reqs = cc.encode_requests(EXAMPLES, encode)
    assert len(reqs) == 6 and reqs[0].continuation_text == "twist the lid"
    r = reqs[0]
    assert bytes(t - 3 for t in r.continuation_ids).decode() == " twist the lid"
    assert len(r.input_ids) == len(encode("Question: open a jar\nAnswer: twist the lid")) - 1
    with pytest.raises(ValueError, match="empty token span"):
        cc.encode_requests([{"goal": "g", "choices": [""], "label": 0}], encode, delimiter="")


def test_scores_do_not_depend_on_batching_here_and_pick_the_liked_choice():
    reqs = cc.encode_requests(EXAMPLES, encode)
    model = favouring(b" twisthelduoawcn")
    a = cc.score_requests(model, reqs, batch_size=2, pad_id=0)
    b = cc.score_requests(model, reqs, batch_size=6, pad_id=0)
    assert a == pytest.approx(b) and all(s < 0 for s in a)
    res = cc.choice_result(EXAMPLES, reqs, a)
    assert res["examples"] == 3 and 0 <= res["accuracy"] <= 1 and len(res["samples"]) == 3
    assert res["accuracy_stderr"] == pytest.approx((res["accuracy"] * (1 - res["accuracy"]) / 3) ** 0.5)
    with pytest.raises(RuntimeError, match="non-finite"):
        cc.score_requests(lambda ids: torch.full((*ids.shape, 260), float("nan")), reqs, batch_size=3, pad_id=0)


def test_results_are_cached_per_identity_and_aggregated(tmp_path):
    bench = tmp_path / "bench.jsonl"
    bench.write_text("\n".join(json.dumps(e) for e in EXAMPLES))
    ident = cc.identity(benchmark_file=bench, tokenizer_sha256="t" * 64, template="Question: {goal}\nAnswer:", delimiter=" ",
                        model_geometry={"layers": 2}, batch_size=4)
    calls = []

    def load(path):
        calls.append(path)
        return favouring(b" twisthelduoawcn" if path == "ckpt-20" else b" eatdig")
    rows = cc.run(tmp_path / "out", {10: "ckpt-10", 20: "ckpt-20"}, load, EXAMPLES, encode, ident, tokens_per_iteration=1000, batch_size=4, pad_id=0)
    assert [r["tokens"] for r in rows] == [10_000, 20_000] and calls == ["ckpt-10", "ckpt-20"]
    assert rows[1]["accuracy_normalised"] > rows[0]["accuracy_normalised"]
    cc.run(tmp_path / "out", {10: "ckpt-10", 20: "ckpt-20", 30: "ckpt-30"}, load, EXAMPLES, encode, ident, tokens_per_iteration=1000, batch_size=4, pad_id=0)
    assert calls == ["ckpt-10", "ckpt-20", "ckpt-30"]                      # only the new checkpoint was scored
    curve = json.loads((tmp_path / "out" / "curve.json").read_text())
    assert curve["identity_sha256"] == ident["sha256"] and len(curve["rows"]) == 3
    other = cc.identity(benchmark_file=bench, tokenizer_sha256="u" * 64, template="Question: {goal}\nAnswer:", delimiter=" ",
                        model_geometry={"layers": 2}, batch_size=4)
    with pytest.raises(ValueError, match="another evaluation identity"):
        cc.load_cached(tmp_path / "out", 10, other, 1000)
    path = cc.result_path(tmp_path / "out", 10)
    body = json.loads(path.read_text())
    body["accuracy"] = 0.99
    path.write_text(json.dumps(body))
    with pytest.raises(ValueError, match="inconsistent"):
        cc.load_cached(tmp_path / "out", 10, ident, 1000)
    with pytest.raises(FileNotFoundError):
        cc.aggregate(tmp_path / "out", [40], ident, 1000)
