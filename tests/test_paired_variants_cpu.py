"""Two variants on the same windows: device reductions, exact aggregation, problem-clustered bootstrap, choice pairing."""
import math

import pytest
import torch

from archlab_b200.evaluation import paired_variants as pv


def test_window_scores_match_direct_computation_and_aggregate_exactly():
    torch.manual_seed(0)
    la, lb = torch.randn(12, 9), torch.randn(12, 9)
    labels = torch.randint(0, 9, (12,))
    labels[::4] = -1
    whole = pv.score_window(la, lb, labels)
    keep = labels >= 0
    assert whole["targets"] == int(keep.sum())
    assert whole["a"]["nll"] == pytest.approx(float(torch.nn.functional.cross_entropy(la[keep], labels[keep], reduction="sum")), rel=1e-5)
    pa, pb = torch.softmax(la[keep], -1), torch.softmax(lb[keep], -1)
    assert whole["a_to_b_kl_sum"] == pytest.approx(float((pa * (pa / pb).log()).sum()), rel=1e-4) and whole["a_to_b_kl_sum"] > 0
    parts = [pv.score_window(la[:6], lb[:6], labels[:6]), pv.score_window(la[6:], lb[6:], labels[6:])]
    one, two = pv.aggregate([whole]), pv.aggregate(parts)
    assert two["windows"] == 2 and one["variants"]["a"]["cross_entropy"] == pytest.approx(two["variants"]["a"]["cross_entropy"], rel=1e-6)
    assert one["token_argmax_agreement"] == two["token_argmax_agreement"] and one["variants"]["b"]["perplexity"] == pytest.approx(math.exp(one["variants"]["b"]["cross_entropy"]))
    same = pv.score_window(la, la, labels)
    assert same["a_to_b_kl_sum"] == pytest.approx(0, abs=1e-6) and same["argmax_agreement_count"] == same["targets"]
    with pytest.raises(ValueError):
        pv.score_window(la, lb, torch.full((12,), -1))


def test_bootstrap_clusters_by_problem():
    torch.manual_seed(1)
    records = []
    for problem in range(12):
        for w in range(3):
            la = torch.randn(10, 7)
            lb = la + 0.8 * torch.nn.functional.one_hot(torch.arange(10) % 7, 7)       # variant b knows the answer better
            r = pv.score_window(la, lb, torch.arange(10) % 7)
            records.append({**r, "problem_sha256": f"p{problem}", "mode": "high" if problem % 2 else "low", "has_tools": problem % 3 == 0})
    s = pv.summary(records, seed=3, replicates=500)
    assert s["paired_uncertainty"]["problem_clusters"] == 12 and set(s["by_mode"]) == {"high", "low"} and set(s["by_tools"]) == {"tools", "no_tools"}
    lo, hi = s["paired_uncertainty"]["cross_entropy_delta_interval"]
    assert lo <= s["overall"]["b_minus_a_ce"] <= hi < 0                                # b is better and the interval excludes zero


def test_choice_pairing():
    case = {"id": "c1", "choices": ["yes", "certainly not"], "answer": 1}
    v = pv.score_choice_vector(case, [-3.0, -6.5])
    assert v["prediction"] == 0 and v["normalized_prediction"] == 1 and v["accuracy"] == 0 and v["accuracy_norm"] == 1
    assert pv.score_choice_vector({**case, "length_normalised": False}, [-3.0, -6.5])["normalized_prediction"] == 0
    with pytest.raises(ValueError, match="non-finite"):
        pv.score_choice_vector(case, [-3.0, float("nan")])
    records = [{"task": "quiz", "id": f"q{i}", "result": {"a": {"prediction": 0, "accuracy": int(i < 3), "accuracy_norm": int(i < 3)},
                                                          "b": {"prediction": int(i > 6), "accuracy": int(i < 6), "accuracy_norm": int(i < 5)}},
                "exact_overlap_consumed_training": i == 2} for i in range(10)]
    out = pv.choice_summary(records)["quiz"]
    assert out["samples"] == 10 and out["accuracy"]["gained"] == 3 and out["accuracy"]["lost"] == 0 and out["prediction_agreement"] == 0.7
    assert out["overlaps_with_consumed_training"] == ["q2"]
