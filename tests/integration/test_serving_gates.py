"""Serving gates: a checkpoint reloaded into the serving engine reproduces the learner's tokens, and the
engine's page pool bounds the context it admits."""
import pytest
import torch

from archlab_b200.models import limite as L
from archlab_b200.serve.engine import SimplicialServingEngine


def _converted(seed=0):
    torch.manual_seed(seed)
    m = L.LimiteLM(L.LimiteConfig.tiny(sliding_window=30))
    m.init_weights(0.2)
    L.replace_limite_attention(m, L.ConversionConfig(short_window=4))
    with torch.no_grad():
        for b in m.layers:
            b.attn.short_kv_delta.normal_(0, 0.05)
    return m.eval()


def test_full_checkpoint_short_context_parity(tmp_path):
    learner = _converted()
    torch.save(learner.state_dict(), tmp_path / "model.pt")
    served = _converted(seed=9)                                   # different weights until the checkpoint is loaded
    served.load_state_dict(torch.load(tmp_path / "model.pt"))
    eng = SimplicialServingEngine(served, num_pages=4, max_batch=2, max_seq_len=256)
    prompt = torch.randint(0, 128, (20,)).tolist()
    rid = eng.add_request(prompt, 5)
    out = eng.run_until_done()[rid]
    seq = list(prompt)
    with torch.no_grad():
        for t in out:
            assert int(learner(torch.tensor([seq]))[0, -1].argmax()) == t
            seq.append(t)


def test_native_context_capacity():
    eng = SimplicialServingEngine(_converted(), num_pages=3, max_batch=4, max_seq_len=256)
    with pytest.raises(ValueError):
        eng.add_request([1] * 250, 10)                           # beyond the engine's sequence limit
    a = eng.add_request([1] * 200, 4)                            # 2 pages
    b = eng.add_request([2] * 150, 4)                            # needs 2 more: must wait for the first to finish
    stats = eng.step()
    assert stats["admitted"] == 1 and stats["waiting"] == 1 and stats["free_pages"] == 1
    out = eng.run_until_done()
    assert len(out[a]) == 4 and len(out[b]) == 4 and len(eng.free) == 3
