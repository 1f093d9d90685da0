"""Full-prefix sampling from a model without an inference cache."""
import json

import pytest
import torch

from archlab_b200.models.qwen38 import Qwen38Config, Qwen38LM
from archlab_b200.train.sample_checkpoint import full_prefix_generate, sample_prompts


def test_greedy_sampling_is_reproducible_and_stops(tmp_path):
    torch.manual_seed(0)
    model = Qwen38LM(Qwen38Config.for_scale("tiny"))
    model.init_weights()
    a = full_prefix_generate(model, [1, 2, 3], max_new_tokens=6)
    b = full_prefix_generate(model, [1, 2, 3], max_new_tokens=6)
    assert a == b and len(a["tokens"]) == 6 and a["finish_reason"] == "length" and model.training
    stop = full_prefix_generate(model, [1, 2, 3], max_new_tokens=6, stop_tokens=(a["tokens"][1],))
    assert stop["finish_reason"] == "stop" and stop["tokens"] == a["tokens"][:2]
    assert full_prefix_generate(model, [1, 2, 3], max_new_tokens=6, max_context=5)["finish_reason"] == "context"
    s1 = full_prefix_generate(model, [1, 2, 3], max_new_tokens=8, temperature=1.0, top_p=0.9, seed=5)
    s2 = full_prefix_generate(model, [1, 2, 3], max_new_tokens=8, temperature=1.0, top_p=0.9, seed=5)
    assert s1 == s2
    with pytest.raises(ValueError):
        full_prefix_generate(model, [], max_new_tokens=2)
    receipt = sample_prompts(model, [[1, 2], [3, 4, 5]], tmp_path / "samples.json", checkpoint="ckpt-10", max_new_tokens=3,
                             decode=lambda ids: " ".join(map(str, ids)))
    saved = json.loads((tmp_path / "samples.json").read_text())
    assert saved == json.loads(json.dumps(receipt)) and len(saved["samples"]) == 2 and saved["optimizer_state_loaded"] is False
    assert saved["samples"][1]["prompt"] == [3, 4, 5] and saved["samples"][0]["text"].count(" ") == 2
