"""Fixed-cache decode controls on CPU (eager decoder path; capture is exercised on a GPU by the same function)."""
import pytest
import torch

from archlab_b200.models.limite import LimiteConfig, LimiteLM, StaticDecodeCache
from archlab_b200.train.qualify_decode import cache_equal, cache_selection_equal, fixed_cache_decode_controls, select_rows


def model():
    torch.manual_seed(0)
    m = LimiteLM(LimiteConfig.tiny())
    m.init_weights(0.05)
    return m.eval()


@pytest.mark.parametrize("teacher_forcing", [True, False])
def test_controls_pass_on_a_correct_implementation(teacher_forcing):
    m = model()
    ids = torch.randint(0, 128, (3, 12 + (6 if teacher_forcing else 0)))
    report = fixed_cache_decode_controls(m, ids, capacity=32, steps=6, teacher_forcing=teacher_forcing)
    assert report["decoder_bitwise_equal"] and report["migration_bitwise_equal"] and report["max_abs_error_vs_full_forward"] < 2e-3
    assert report["prompt_tokens"] == 12 and report["captured"] is False


def test_controls_catch_indexing_errors():
    m = model()
    c = m.config
    a, b = StaticDecodeCache(c, 2, 16, "cpu", torch.float32), StaticDecodeCache(c, 2, 16, "cpu", torch.float32)
    ks = [torch.randn(2, 10, c.num_key_value_heads, c.head_dim) for _ in range(c.num_hidden_layers)]
    a.load_prefill(ks, ks), b.load_prefill(ks, ks)
    assert cache_equal(a, b)
    b.k[1][0, 3] += 1
    assert not cache_equal(a, b)
    rows = torch.tensor([1])
    moved = select_rows(a, rows)
    assert cache_selection_equal(a, moved, rows)
    moved.v[0][0, int(a.position) % a.sizes[0] - 1] += 1                           # a visible slot of a local layer
    assert not cache_selection_equal(a, moved, rows)
    with pytest.raises(ValueError, match="fit the cache"):
        fixed_cache_decode_controls(m, torch.randint(0, 128, (1, 30)), capacity=32, steps=6, teacher_forcing=False)
    with pytest.raises(ValueError, match="eval mode"):
        fixed_cache_decode_controls(m.train(), torch.randint(0, 128, (1, 10)), capacity=32)
