"""CORE task types: rendering, spans, verdicts with an oracle 'model'."""
import pytest
import torch

from archlab_b200.evaluation import core_tasks as ct


def encode(text):
    return [1] + [2 + b for b in text.encode()]


def oracle(truth: str):
    """Predicts the next byte of ``truth`` wherever the input is a prefix of it; uniform elsewhere."""
    target = encode(truth)

    def logits(ids):
        out = torch.zeros(*ids.shape, 260)
        for r in range(ids.shape[0]):
            row = ids[r].tolist()
            for t in range(len(row)):
                if row[:t + 1] == target[:t + 1] and t + 1 < len(target):
                    out[r, t, target[t + 1]] = 10.0
        return out
    return logits


def test_rendering_and_spans():
    mc = {"query": "2+2=", "choices": ["4", "5"], "gold": 0}
    shots = [{"query": "1+1=", "choices": ["2", "3"], "gold": 0}]
    assert ct.render_prompts(mc, "multiple_choice", " ", shots) == ["1+1= 2\n\n2+2= 4", "1+1= 2\n\n2+2= 5"]
    sc = {"context_options": ["The cat", "The rock"], "continuation": "purrs", "gold": 0}
    assert ct.render_prompts(sc, "schema", " ") == ["The cat purrs", "The rock purrs"]
    lm = {"context": "Paris is in  ", "continuation": "France"}
    assert ct.render_prompts(lm, "language_modeling", " ") == ["Paris is in", "Paris is in France"]
    assert ct.common_length([[1, 2, 3], [1, 2, 4]]) == 2 and ct.common_length([[9, 2, 3], [7, 8, 2, 3]], "right") == 2
    seqs, starts, ends = ct.token_spans("schema", [encode("The cat purrs"), encode("The rock purrs")])
    assert [e - s for s, e in zip(starts, ends)] == [len(" purrs")] * 2
    with pytest.raises(ValueError, match="token prefix"):
        ct.token_spans("language_modeling", [[1, 2, 9], [1, 2, 3, 4]])
    with pytest.raises(ValueError, match="unknown task type"):
        ct.render_prompts(mc, "cloze", " ")


def test_verdicts_follow_the_model():
    mc = {"query": "2+2=", "choices": ["5", "4"], "gold": 1}
    assert ct.evaluate_item(oracle("2+2= 4"), encode, mc, "multiple_choice") and not ct.evaluate_item(oracle("2+2= 5"), encode, mc, "multiple_choice")
    sc = {"context_options": ["The rock", "The cat"], "continuation": "purrs", "gold": 1}
    assert ct.evaluate_item(oracle("The cat purrs"), encode, sc, "schema") and not ct.evaluate_item(oracle("The rock purrs"), encode, sc, "schema")
    lm = {"context": "Paris is in ", "continuation": "France"}
    assert ct.evaluate_item(oracle("Paris is in France"), encode, lm, "language_modeling")
    assert not ct.evaluate_item(oracle("Paris is in Franca"), encode, lm, "language_modeling")            # one wrong token fails the exact match
    target = encode("Paris is in France")

    def windowed(ids):                                                          # finds the cropped window inside the truth
        out = torch.zeros(*ids.shape, 260)
        row = ids[0].tolist()
        cut = len(target) - len(row)
        assert row == target[cut:]
        for t in range(len(row) - 1):
            out[0, t, target[cut + t + 1]] = 10.0
        return out
    assert ct.evaluate_item(windowed, encode, lm, "language_modeling", max_tokens=12)                     # left-cropped prompt, shifted span
    with pytest.raises(ValueError, match="does not fit"):
        ct.evaluate_item(oracle("Paris is in France"), encode, lm, "language_modeling", max_tokens=5)


def test_task_loop_strides_ranks_and_draws_fewshot_deterministically():
    data = [{"query": f"{i}+0=", "choices": [str(i), str(i + 1)], "gold": 0} for i in range(6)]
    meta = {"task_type": "multiple_choice", "num_fewshot": 2, "continuation_delimiter": " "}
    seen = []

    def spy(ids):
        seen.append(ids.shape)
        return torch.zeros(*ids.shape, 260)
    a = ct.evaluate_task(spy, encode, data, meta, rank=0, world=2)
    b = ct.evaluate_task(spy, encode, data, meta, rank=1, world=2)
    assert a[1] == b[1] == 3 and len(seen) == 6 and all(s[0] == 2 for s in seen)
    first = list(seen)
    seen.clear()
    ct.evaluate_task(spy, encode, data, meta, rank=0, world=2)
    assert seen == first[:3]                                                   # same few-shot draws on a re-run
    with pytest.raises(ValueError, match="unknown task type"):
        ct.evaluate_task(spy, encode, data, {"task_type": "cloze"})


def test_bundle_directory_to_centred_metric(tmp_path):
    import json

    (tmp_path / "eval_data").mkdir()
    (tmp_path / "core.yaml").write_text(
        "icl_tasks:\n"
        "- {label: sums, icl_task_type: multiple_choice, dataset_uri: sums.jsonl, num_fewshot: [0]}\n"
        "- {label: capitals, icl_task_type: language_modeling, dataset_uri: cap.jsonl, num_fewshot: [0], continuation_delimiter: ' '}\n")
    (tmp_path / "eval_meta_data.csv").write_text("Eval Task,Random baseline\nsums,50\ncapitals,0\n")
    (tmp_path / "eval_data" / "sums.jsonl").write_text("\n".join(json.dumps({"query": "2+2=", "choices": ["5", "4"], "gold": g}) for g in (1, 0)) + "\n")
    (tmp_path / "eval_data" / "cap.jsonl").write_text(json.dumps({"context": "Paris is in", "continuation": "France"}) + "\n")
    tasks = ct.read_bundle(tmp_path)
    assert [t["label"] for t in tasks] == ["sums", "capitals"] and tasks[0]["random_baseline"] == 0.5

    both = oracle("2+2= 4")
    out = ct.evaluate_bundle(both, encode, tasks)
    assert out["results"] == {"sums": 0.5, "capitals": 0.0}                     # the model says 4: right for gold=1, wrong for gold=0
    assert out["centered_results"] == {"sums": 0.0, "capitals": 0.0} and out["core_metric"] == 0.0
    assert ct.evaluate_bundle(both, encode, tasks, max_per_task=1)["results"]["sums"] in (0.0, 1.0)

    (tmp_path / "eval_meta_data.csv").write_text("Eval Task,Random baseline\nsums,50\n")
    with pytest.raises(ValueError, match="capitals: no random baseline"):
        ct.read_bundle(tmp_path)
