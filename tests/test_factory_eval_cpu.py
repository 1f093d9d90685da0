import math

import pytest
import torch

from archlab_b200.models import factory
from archlab_b200.train import evaluation as ev


def test_factory_builds_every_family_and_patches_legacy_config():
    assert {"nanochat", "kimi_kda", "qwen35", "deepseek_v41", "qwen38_27b_text"} <= set(factory.families())
    m = factory.build_model("kimi_kda", dict(vocab_size=64, n_layer=2, n_head=2, n_embd=16, legacy_flag=True))
    assert m.config.n_embd == 16 and sum(p.numel() for p in m.parameters()) > 0
    patched = factory.patch_config("kimi_kda", {"n_embd": 16, "removed_key": 1})
    assert patched["__dropped__"] == ["removed_key"]
    with pytest.raises(ValueError):
        factory.classes_for("nope")
    q = factory.build_from_meta({"model_config": {"arch_family": "qwen38_tiny", "vocab_size": 128, "sequence_len": 16,
                                                  "num_hidden_layers": 2, "hidden_size": 32, "intermediate_size": 64,
                                                  "attention_heads": 2, "attention_kv_heads": 1, "attention_head_dim": 16,
                                                  "linear_qk_heads": 1, "linear_v_heads": 2, "linear_key_dim": 8,
                                                  "linear_value_dim": 8, "eos_token_id": 0}})
    assert q.config.hidden_size == 32


class _Uniform(torch.nn.Module):
    def __init__(self, V):
        super().__init__()
        self.V = V
        self.p = torch.nn.Parameter(torch.zeros(1))

    def forward(self, x, y=None):
        return torch.zeros(*x.shape, self.V) + self.p


def test_bpb_of_uniform_model_is_log2_vocab_over_bytes():
    V = 16
    m = _Uniform(V)
    token_bytes = torch.full((V,), 2)
    token_bytes[0] = 0                                   # special token: excluded
    x = torch.randint(1, V, (2, 9))
    y = torch.randint(1, V, (2, 9))
    y[0, 0] = -1
    bpb = ev.evaluate_bpb(m, [(x, y)], token_bytes)
    assert abs(bpb - math.log2(V) / 2) < 1e-6


def test_multiple_choice_and_generation():
    torch.manual_seed(0)
    m = factory.build_model("kimi_kda", dict(vocab_size=32, n_layer=2, n_head=2, n_embd=16))
    assert ev.score_multiple_choice(m, [1, 2, 3], [[4, 5], [6, 7], [8]]) in (0, 1, 2)
    outs = ev.generate_batch(m, [[1, 2, 3], [4]], 5)
    assert [len(o) for o in outs] == [5, 5]
    again = ev.generate_batch(m, [[1, 2, 3], [4]], 5)
    assert outs == again
