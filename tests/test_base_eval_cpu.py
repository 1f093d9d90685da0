"""Base-model evaluation modes on a tiny speedrun model."""
import pytest
import torch

from archlab_b200.models.nanochat import GPT, GPTConfig
from archlab_b200.train.base_eval import evaluate_checkpoint, parse_modes, part_batches


def tiny():
    torch.manual_seed(0)
    cfg = GPTConfig(sequence_len=32, vocab_size=64, n_layer=2, n_head=2, n_kv_head=2, n_embd=32)
    m = GPT(cfg)
    m.init_weights()
    return m


def test_modes_are_explicit():
    assert parse_modes("core, bpb") == {"core", "bpb"}
    for bad in ("core,perplexity", ""):
        with pytest.raises(ValueError, match="invalid evaluation modes"):
            parse_modes(bad)


def test_each_mode_runs_and_missing_inputs_are_errors():
    m = tiny()
    tasks = {"toy": {"random_baseline": 0.5, "items": [{"prefix": [1, 2, 3], "choices": [[4, 5], [6]], "gold": 0}, {"prefix": [7], "choices": [[8], [9, 10]], "gold": 1}]}}
    part = torch.arange(4000) % 64
    token_bytes = torch.ones(64, dtype=torch.long)
    token_bytes[0] = 0
    out = evaluate_checkpoint(m, {"core", "bpb", "sample"}, tasks=tasks, bpb_batches={"val": part_batches(part, 2, 32, 1000, "cpu")}, token_bytes=token_bytes,
                              prompts=[[1, 2], [3, 4, 5]], sample_tokens=4, decode=lambda ids: " ".join(map(str, ids)))
    assert set(out) == {"core", "bpb", "samples"} and 0 <= out["core"]["results"]["toy"] <= 1 and 3 < out["bpb"]["val"] < 12
    assert len(out["samples"]) == 2 and len(out["samples"][0]["tokens"]) == 4 and out["samples"][1]["text"].startswith("3 4 5")
    assert set(evaluate_checkpoint(m, {"core"}, tasks=tasks)) == {"core"}
    assert "samples" not in evaluate_checkpoint(m, {"sample"}, prompts=[[1]], rank=1)
    for modes, message in (({"core"}, "task bundle"), ({"bpb"}, "token_bytes"), ({"sample"}, "prompts")):
        with pytest.raises(ValueError, match=message):
            evaluate_checkpoint(m, modes)
    batches = list(part_batches(part, 2, 32, 200, "cpu"))
    assert len(batches) == 3 and torch.equal(batches[0][1][0, :-1], batches[0][0][0, 1:])


def test_core_mode_accepts_the_published_bundle_layout(tmp_path):
    import json

    from archlab_b200.evaluation.core_tasks import read_bundle

    (tmp_path / "eval_data").mkdir()
    (tmp_path / "core.yaml").write_text("icl_tasks:\n- {label: t, icl_task_type: schema, dataset_uri: t.jsonl, num_fewshot: [1]}\n")
    (tmp_path / "eval_meta_data.csv").write_text("Eval Task,Random baseline\nt,50\n")
    (tmp_path / "eval_data" / "t.jsonl").write_text("\n".join(json.dumps({"context_options": [f"a{i}", f"b{i}"], "continuation": "cd", "gold": i % 2}) for i in range(4)) + "\n")
    m = tiny()
    out = evaluate_checkpoint(m, {"core"}, tasks=read_bundle(tmp_path), core_encode=lambda s: [1] + [2 + b % 60 for b in s.encode()], core_max_tokens=32)
    assert set(out["core"]) == {"results", "centered_results", "core_metric"} and 0.0 <= out["core"]["results"]["t"] <= 1.0
