"""KV-cache engine of the speedrun GPT: cached logits equal the full forward pass; sampling API."""
import pytest
import torch

from archlab_b200.models.nanochat import GPT, GPTConfig
from archlab_b200.serve.kv_engine import Engine, KVCache, forward_cached


def _model(pattern="SL"):
    torch.manual_seed(0)
    cfg = GPTConfig(sequence_len=512, vocab_size=300, n_layer=4, n_head=4, n_kv_head=2, n_embd=64, window_pattern=pattern)
    m = GPT(cfg)
    m.init_weights()
    with torch.no_grad():                                   # make the gates and gains matter
        m.smear_lambda.fill_(0.7)
        m.x0_lambdas.uniform_(-0.2, 0.2)
        for p in m.parameters():
            if p.dim() >= 2 and float(p.abs().max()) == 0:
                p.normal_(std=0.05)
    return m.eval()


@pytest.mark.parametrize("split", [(200,), (1, 199), (150, 1, 1, 48), (64, 64, 72)])
def test_cached_logits_equal_full_forward(split):
    m = _model()
    ids = torch.randint(0, 300, (2, sum(split)))
    want = m(ids)
    cache = KVCache(m, 2, 256)
    got, s = [], 0
    for n in split:
        got.append(forward_cached(m, ids[:, s: s + n], cache))
        s += n
    torch.testing.assert_close(torch.cat(got, 1), want, atol=2e-4, rtol=1e-4)
    assert cache.pos == sum(split)


def test_greedy_generation_matches_the_uncached_sampler_and_samples_share_the_prefill():
    m = _model("L")
    prompt = [5, 17, 200, 3]
    eng = Engine(m)
    cached = eng.generate_batch(prompt, max_tokens=12, temperature=0.0)[0]
    naive = prompt + list(m.generate(prompt, 12, temperature=0.0))
    assert cached == naive
    outs = eng.generate_batch(prompt, num_samples=3, max_tokens=8, temperature=1.0, top_k=20, seed=1)
    assert len(outs) == 3 and all(o[:4] == prompt and len(o) == 12 for o in outs) and len({tuple(o) for o in outs}) > 1
    stopped = eng.generate_batch(prompt, max_tokens=12, temperature=0.0, stop_tokens=(cached[6],))[0]
    assert stopped == cached[:6]


def test_engine_refuses_families_with_their_own_trunk():
    from archlab_b200.models.nanochat_variants import MhcGPT, MhcGPTConfig

    m = MhcGPT(MhcGPTConfig(sequence_len=64, vocab_size=64, n_layer=2, n_head=2, n_kv_head=2, n_embd=32))
    with pytest.raises(TypeError):
        Engine(m)


def test_chat_front_is_answered_by_the_engine():
    import json
    import threading
    import urllib.request

    from archlab_b200.data.tokenizer import BPETokenizer
    from archlab_b200.serve.kv_engine import answer_tickets, render_chat
    from archlab_b200.services.chat import ChatFront

    tok = BPETokenizer.train(["hello world, hello there. the quick brown fox"] * 4, vocab_size=280)
    ids = render_chat(tok, [{"role": "system", "content": "be brief"}, {"role": "user", "content": "hello"}])
    assert ids[0] == tok.special["<|bos|>"] and ids[-1] == tok.special["<|assistant_start|>"]
    assert tok.decode(ids[2:-2]) == "be brief\n\nhello"
    torch.manual_seed(0)
    m = GPT(GPTConfig(sequence_len=128, vocab_size=300, n_layer=2, n_head=2, n_kv_head=2, n_embd=32, window_pattern="L"))
    m.init_weights()
    front = ChatFront("127.0.0.1", 0, "tok", {"tiny": "normal"})
    port = front.server.server_address[1]
    stop = threading.Event()
    result = {}

    def client():
        body = json.dumps({"model": "tiny", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 6}).encode()
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=body,
                                     headers={"Authorization": "Bearer tok", "Content-Type": "application/json"})
        result["reply"] = json.loads(urllib.request.urlopen(req, timeout=30).read())
        stop.set()

    t = threading.Thread(target=client)
    t.start()
    served = answer_tickets(front, Engine(m), tok, stop=stop.is_set)
    t.join(10)
    front.server.shutdown()
    assert served == 1 and result["reply"]["object"] == "chat.completion"
    assert isinstance(result["reply"]["choices"][0]["message"]["content"], str)


def test_streamed_reply_equals_the_whole_reply():
    """With ``stream`` the engine's worker emits the reply piece by piece; the pieces concatenate to the same text the
    non-streaming request returns for the same seed."""
    import json
    import threading
    import urllib.request

    from archlab_b200.data.tokenizer import BPETokenizer
    from archlab_b200.serve.kv_engine import answer_tickets
    from archlab_b200.services.chat import ChatFront

    tok = BPETokenizer.train(["hello world, hello there. the quick brown fox"] * 4, vocab_size=280)
    torch.manual_seed(0)
    m = GPT(GPTConfig(sequence_len=128, vocab_size=300, n_layer=2, n_head=2, n_kv_head=2, n_embd=32, window_pattern="L"))
    m.init_weights()
    front = ChatFront("127.0.0.1", 0, "tok", {"tiny": "normal"})
    port = front.server.server_address[1]
    stop = threading.Event()
    got = {}

    def ask(stream):
        body = json.dumps({"model": "tiny", "messages": [{"role": "user", "content": "hello"}], "max_tokens": 8, "seed": 5,
                           "stream": stream}).encode()
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=body,
                                     headers={"Authorization": "Bearer tok", "Content-Type": "application/json"})
        return urllib.request.urlopen(req, timeout=30).read().decode()

    def client():
        got["whole"] = json.loads(ask(False))["choices"][0]["message"]["content"]
        events = [e[len("data: "):] for e in ask(True).split("\n\n") if e.startswith("data: ")]
        got["pieces"] = [json.loads(e)["choices"][0]["delta"].get("content", "") for e in events[:-1]]
        got["last"] = events[-1]
        stop.set()

    t = threading.Thread(target=client)
    t.start()
    served = answer_tickets(front, Engine(m), tok, stop=stop.is_set)
    t.join(10)
    front.server.shutdown()
    assert served == 2 and got["last"] == "[DONE]" and "".join(got["pieces"]) == got["whole"]


def test_nucleus_sampling_keeps_the_smallest_sufficient_set():
    import pytest
    import torch

    from archlab_b200.serve.kv_engine import sample_next

    logits = torch.log(torch.tensor([[0.5, 0.3, 0.15, 0.05]]))
    rng = torch.Generator().manual_seed(0)
    draws = {int(sample_next(logits, 1.0, None, rng, top_p=0.7)) for _ in range(200)}
    assert draws == {0, 1}                                     # 0.5 alone is short of 0.7; 0.5 + 0.3 reaches it
    assert {int(sample_next(logits, 1.0, None, rng, top_p=0.4)) for _ in range(50)} == {0}
    assert {int(sample_next(logits, 1.0, None, rng, top_p=1.0)) for _ in range(400)} == {0, 1, 2, 3}
    assert int(sample_next(logits, 0.0, None, None, top_p=0.1)) == 0
    with pytest.raises(RuntimeError, match="non-finite"):
        sample_next(torch.tensor([[0.0, float("nan")]]), 1.0, None, rng)
