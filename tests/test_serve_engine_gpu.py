"""Serving engine on the GPU: prefill through the simplicial forward kernel, batched decode through its paged
decode mode; greedy tokens agree with full re-computation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_engine_generates_like_full_recomputation():
    from archlab_b200.models import limite as L
    from archlab_b200.ops import native
    from archlab_b200.serve.engine import SimplicialServingEngine

    torch.manual_seed(0)
    cfg = L.LimiteConfig.tiny(vocab_size=512, hidden_size=256, num_attention_heads=4, num_key_value_heads=1, head_dim=128,
                              intermediate_size=512, sliding_window=255, global_layers=(3,))
    m = L.LimiteLM(cfg)
    m.init_weights(0.08)
    L.replace_limite_attention(m, L.ConversionConfig(short_window=8))
    with torch.no_grad():
        for b in m.layers:
            b.attn.short_kv_delta.normal_(0, 0.02)
    m = m.cuda().bfloat16().eval()
    eng = SimplicialServingEngine(m, num_pages=16, max_batch=4, max_seq_len=512)
    prompts = [torch.randint(0, 512, (n,)).tolist() for n in (256, 128, 384)]
    ids = [eng.add_request(p, 8) for p in prompts]
    out = eng.run_until_done()
    native.check_status()
    agree = total = 0
    with torch.no_grad():
        for rid, p in zip(ids, prompts):
            seq = list(p)
            for t in out[rid]:                                   # teacher-forced check: bf16 ties may flip an argmax
                pad = (-len(seq)) % 128
                logits = m(torch.tensor([seq + [0] * pad], device="cuda"))[0, len(seq) - 1]
                top2 = logits.topk(2).values
                agree += int(int(logits.argmax()) == t or float(top2[0] - logits[t]) < 0.05 * float(top2[0].abs() + 1))
                total += 1
                seq.append(t)
    assert agree == total and len(eng.free) == 16
