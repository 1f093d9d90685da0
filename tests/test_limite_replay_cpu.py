"""Limite long-context replay: same values and gradients as the plain forward, fewer retained activations, one shared
context that refuses cold geometries once locked."""
import pytest
import torch

from archlab_b200.models.limite import AdapterConfig, LimiteConfig, LimiteLM, install_adapters
from archlab_b200.models.limite_replay import (ReplayContextCache, bounded_window_attention, replay_hidden, replay_loss,
                                               retained_activation_bytes)
from archlab_b200.ops.trunk import attention_reference


def _model(adapters=False):
    torch.manual_seed(0)
    m = LimiteLM(LimiteConfig.tiny())
    m.init_weights(0.05)
    if adapters:
        install_adapters(m, AdapterConfig())
    return m


@pytest.mark.parametrize("window", [-1, 0, 5, 40])
def test_bounded_attention_matches_the_definition(window):
    torch.manual_seed(1)
    q, k, v = torch.randn(2, 37, 4, 8, requires_grad=True), torch.randn(2, 37, 2, 8, requires_grad=True), torch.randn(2, 37, 2, 8, requires_grad=True)
    want = attention_reference(q, k, v, window)
    got = bounded_window_attention(q, k, v, window, query_tile=8)
    assert torch.allclose(got, want, atol=1e-5)
    g = torch.randn_like(want)
    a = torch.autograd.grad(want, (q, k, v), g)
    b = torch.autograd.grad(got, (q, k, v), g)
    assert all(torch.allclose(x, y, atol=1e-5) for x, y in zip(a, b))


def _saved_bytes(fn):
    total = [0]

    def pack(t):
        total[0] += t.numel() * t.element_size()
        return t
    with torch.autograd.graph.saved_tensors_hooks(pack, lambda t: t):
        out = fn()
    return out, total[0]


def test_replay_equals_the_plain_forward_and_retains_less():
    model = _model()
    ids = torch.randint(0, 128, (2, 48))
    want, plain_bytes = _saved_bytes(lambda: model.hidden(ids))
    got, replay_bytes = _saved_bytes(lambda: replay_hidden(model, ids, query_tile=16))
    assert torch.allclose(got, want, atol=1e-5) and replay_bytes < 0.5 * plain_bytes
    g = torch.randn_like(want)
    want.backward(g)
    reference = {n: p.grad.clone() for n, p in model.named_parameters() if p.grad is not None}
    model.zero_grad()
    got.backward(g)
    assert all(float((p.grad - reference[n]).abs().max()) <= 1e-5 + 2e-6 * float(reference[n].abs().max()) for n, p in model.named_parameters() if n in reference)
    c = model.config
    assert retained_activation_bytes(c, 2, 48) < 0.25 * retained_activation_bytes(c, 2, 48, checkpoint_layers=False)


def test_replay_loss_matches_cross_entropy_with_ignored_labels():
    model = _model()
    ids = torch.randint(0, 128, (2, 20))
    labels = ids.roll(-1, 1).clone()
    labels[:, -3:] = -1
    out = replay_loss(model, ids, labels, chunk_size=7, query_tile=8)
    want = model(ids, labels)
    assert torch.allclose(out["loss"], want, atol=1e-5) and out["tokens"] == 34 and float(out["entropy"]) > 0
    out["loss"].backward()
    assert model.lm_head.weight.grad is not None


def test_context_is_built_once_and_locked_against_cold_keys():
    model = _model()
    cache = ReplayContextCache()
    ids = torch.randint(0, 128, (1, 16))
    with pytest.raises(RuntimeError, match="enable"):
        cache.prepare(model, ids)
    cache.enable()
    first = cache.prepare(model, ids)
    replay_hidden(model, ids, cache=cache)
    replay_hidden(model, torch.randint(0, 128, (1, 16)), cache=cache)        # other tokens, same geometry
    assert cache.prepare(model, ids) is first and cache.builds == 1
    cache.lock()
    replay_hidden(model, ids, cache=cache)
    with pytest.raises(RuntimeError, match="before capture"):
        replay_hidden(model, torch.randint(0, 128, (1, 24)), cache=cache)
    model.eval()
    with pytest.raises(RuntimeError, match="before capture"):               # train/eval is part of the key
        cache.prepare(model, ids)
    cache.enable(False)
    assert cache.entry is None and not cache.locked
