"""KV-cache inference engine for the speedrun GPT: prefill once, then one token per step for a batch of samples.

The reference's ``Engine`` (src/archlab/speedrun/engine.py) prefills the prompt with batch 1, clones the cache for
``num_samples`` rows and decodes them together; chat and the sampling evaluations sit on it.  Here the cache is one
pre-sized tensor pair per layer (``[rows, capacity, kv heads, head dim]``, written in place, so decode steps allocate
nothing that grows), the smear gate keeps the previous token's embedding, and windowed layers only read the last
``window + 1`` cache positions.  ``forward_cached`` reproduces ``GPT.forward`` position by position: prefill +
decode logits equal the logits of one full forward pass.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from ..models.nanochat import GPT, apply_rope, rms_norm


class KVCache:
    def __init__(self, model: GPT, rows: int, capacity: int, device=None, dtype=None):
        cfg = model.config
        device = device or model.transformer.wte.weight.device
        dtype = dtype or cfg.compute_dtype
        if capacity > model.cos.size(0):
            raise ValueError(f"capacity {capacity} exceeds the rotary table of {model.cos.size(0)} positions")
        shape = (rows, capacity, cfg.n_kv_head, cfg.head_dim)
        self.k = [torch.zeros(shape, device=device, dtype=dtype) for _ in range(cfg.n_layer)]
        self.v = [torch.zeros(shape, device=device, dtype=dtype) for _ in range(cfg.n_layer)]
        self.pos = 0
        self.prev_embedding = None          # normalised embedding of the last token seen (smear gate)
        self.rows, self.capacity = rows, capacity

    def expanded(self, rows: int) -> "KVCache":
        """A cache of ``rows`` rows holding copies of this single-row cache (prompt prefilled once, sampled many times)."""
        if self.rows != 1:
            raise ValueError("only a single-row cache can be expanded")
        new = object.__new__(KVCache)
        new.k = [t.expand(rows, -1, -1, -1).clone() for t in self.k]
        new.v = [t.expand(rows, -1, -1, -1).clone() for t in self.v]
        new.pos, new.rows, new.capacity = self.pos, rows, self.capacity
        new.prev_embedding = None if self.prev_embedding is None else self.prev_embedding.expand(rows, -1, -1).clone()
        return new


def _attend(q, k, v, q0: int, window: int):
    """q [B,T,H,D] at absolute positions q0..q0+T-1 against cache rows 0..q0+T-1 (left window, -1 = unlimited)."""
    T, K = q.size(1), k.size(1)
    qpos = torch.arange(q0, q0 + T, device=q.device).view(T, 1)
    kpos = torch.arange(K, device=q.device).view(1, K)
    mask = kpos <= qpos
    if window >= 0:
        mask = mask & ((qpos - kpos) <= window)
    y = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask,
                                       enable_gqa=q.size(2) != k.size(2))
    return y.transpose(1, 2)


@torch.no_grad()
def forward_cached(model: GPT, idx: torch.Tensor, cache: KVCache) -> torch.Tensor:
    """Logits [B, T, vocab] for ``idx`` appended to the cached prefix; the cache advances by T."""
    cfg = model.config
    B, T = idx.shape
    p0 = cache.pos
    if p0 + T > cache.capacity:
        raise ValueError("the cache is full")
    cos, sin = model.cos[p0: p0 + T], model.sin[p0: p0 + T]
    x = rms_norm(model.transformer.wte(idx).to(cfg.compute_dtype))
    G = model.smear_gate_channels
    prev = torch.cat([x[:, :1] * 0 if cache.prev_embedding is None else cache.prev_embedding, x[:, :-1]], 1)
    gate = model.smear_lambda.to(x.dtype) * torch.sigmoid(model.smear_gate(x[..., :G]))
    if cache.prev_embedding is None:
        gate = torch.cat([gate[:, :1] * 0, gate[:, 1:]], 1)            # the very first token has nothing to smear in
    cache.prev_embedding = x[:, -1:].clone()
    x = x + gate * prev
    x0, x_backout = x, None
    for i, block in enumerate(model.transformer.h):
        x = model.resid_lambdas[i].to(x.dtype) * x + model.x0_lambdas[i].to(x.dtype) * x0
        a = block.attn
        h = rms_norm(x)
        q = a.c_q(h).view(B, T, cfg.n_head, cfg.head_dim)
        k = a.c_k(h).view(B, T, cfg.n_kv_head, cfg.head_dim)
        v = a.c_v(h).view(B, T, cfg.n_kv_head, cfg.head_dim)
        if str(i) in model.value_embeds:
            ve = model.value_embeds[str(i)](idx).to(x.dtype)
            v = v + (3 * torch.sigmoid(a.ve_gate(h[..., : a.ve_gate_channels]))).unsqueeze(-1) * ve.view_as(v)
        q, k = rms_norm(apply_rope(q, cos, sin)) * 1.2, rms_norm(apply_rope(k, cos, sin)) * 1.2
        cache.k[i][:, p0: p0 + T] = k
        cache.v[i][:, p0: p0 + T] = v
        w = model.window_sizes[i]
        lo = 0 if w < 0 else max(0, p0 - w)                           # windowed layers never look further back
        y = _attend(q, cache.k[i][:, lo: p0 + T], cache.v[i][:, lo: p0 + T], p0 - lo, w)
        x = x + a.c_proj(y.contiguous().view(B, T, -1))
        x = x + block.mlp(rms_norm(x))
        if i == cfg.n_layer // 2:
            x_backout = x
    if x_backout is not None:
        x = x - model.backout_lambda.to(x.dtype) * x_backout
    cache.pos = p0 + T
    logits = model.lm_head(rms_norm(x))[..., : cfg.vocab_size].float()
    return cfg.logit_softcap * torch.tanh(logits / cfg.logit_softcap)


def sample_next(logits: torch.Tensor, temperature: float, top_k: int | None, rng, top_p: float = 1.0) -> torch.Tensor:
    """logits [B, V] -> token ids [B, 1]; temperature 0 is greedy.  ``top_p`` < 1 keeps the smallest set of most probable
    tokens whose mass reaches ``top_p`` (the token that crosses the threshold is kept, so the set is never empty).
    Non-finite logits are an error rather than a sample."""
    if not torch.isfinite(logits).all():
        raise RuntimeError("sampling logits contain non-finite values")
    if temperature <= 0:
        return logits.argmax(-1, keepdim=True)
    if top_k:
        kth = logits.topk(min(top_k, logits.size(-1)), dim=-1).values[:, -1:]
        logits = logits.masked_fill(logits < kth, float("-inf"))
    probabilities = F.softmax(logits / temperature, dim=-1)
    if top_p < 1.0:
        ordered, index = probabilities.sort(descending=True, dim=-1)
        ordered = ordered.masked_fill(ordered.cumsum(-1) - ordered > top_p, 0.0)       # mass BEFORE the token already exceeds top_p
        return index.gather(-1, torch.multinomial(ordered, 1, generator=rng))
    return torch.multinomial(probabilities, 1, generator=rng)


class Engine:
    def __init__(self, model: GPT):
        if type(model).trunk is not GPT.trunk:
            raise TypeError("the cached engine reproduces the plain speedrun trunk; this family overrides it")
        self.model = model

    @torch.no_grad()
    def generate(self, tokens: list[int], *, num_samples: int = 1, max_tokens: int = 64, temperature: float = 1.0,
                 top_k: int | None = None, seed: int = 42, stop_tokens: tuple[int, ...] = (), top_p: float = 1.0):
        """Yields ``(column, done)`` per step: ``column[r]`` is the token sample ``r`` produced (None once it has
        stopped) and ``done[r]`` whether it has stopped.  The prompt is prefilled once and shared by all samples."""
        model = self.model
        was_training = model.training
        model.eval()
        dev = model.transformer.wte.weight.device
        rng = torch.Generator(device=dev).manual_seed(seed) if temperature > 0 else None
        capacity = min(model.cos.size(0), len(tokens) + max_tokens)
        base = KVCache(model, 1, capacity)
        logits = forward_cached(model, torch.tensor([tokens], dtype=torch.long, device=dev), base)[:, -1]
        cache = base.expanded(num_samples) if num_samples > 1 else base
        logits = logits.expand(num_samples, -1)
        done = [False] * num_samples
        try:
            for _ in range(max_tokens):
                nxt = sample_next(logits, temperature, top_k, rng, top_p)
                column = []
                for r, t in enumerate(nxt[:, 0].tolist()):
                    column.append(None if done[r] else t)
                    done[r] = done[r] or t in stop_tokens
                yield column, list(done)
                if all(done) or cache.pos >= cache.capacity:
                    break
                logits = forward_cached(model, nxt, cache)[:, -1]
        finally:
            model.train(was_training)

    def generate_batch(self, tokens: list[int], **kw) -> list[list[int]]:
        """The completed sequences (prompt + generated tokens up to and excluding a stop token) of every sample."""
        out = [list(tokens) for _ in range(kw.get("num_samples", 1))]
        stops = set(kw.get("stop_tokens", ()))
        for column, _ in self.generate(tokens, **kw):
            for r, t in enumerate(column):
                if t is not None and t not in stops:
                    out[r].append(t)
        return out


# ------------------------------------------------------------------------------------------------
# chat: conversation -> tokens, and the worker that answers the tickets of the HTTP front
# ------------------------------------------------------------------------------------------------
def render_chat(tokenizer, messages: list[dict]) -> list[int]:
    """``<|bos|>`` then every turn between its role markers (a system message is folded into the first user turn),
    ending with ``<|assistant_start|>`` so that the model writes the reply (speedrun chat format,
    src/archlab/speedrun/tokenizer.py ``render_for_completion``)."""
    sp = tokenizer.special
    ids = [sp["<|bos|>"]]
    pending = ""
    for m in messages:
        if m["role"] == "system":
            pending += m["content"] + "\n\n"
            continue
        role = "user" if m["role"] == "user" else "assistant"
        text = (pending + m["content"]) if role == "user" else m["content"]
        pending = "" if role == "user" else pending
        ids += [sp[f"<|{role}_start|>"], *tokenizer.encode(text), sp[f"<|{role}_end|>"]]
    return ids + [sp["<|assistant_start|>"]]


def answer_tickets(front, engine: "Engine", tokenizer, *, stop=None, idle_timeout: float = 0.2, top_k: int | None = 50) -> int:
    """Drains the chat front's ticket queue on the thread that owns the model until ``stop()`` is true: one
    generation per ticket, reply text = decoded tokens up to ``<|assistant_end|>``.  Returns the tickets served."""
    served = 0
    end = tokenizer.special["<|assistant_end|>"]
    while not (stop and stop()):
        ticket = front.next_ticket(timeout=idle_timeout)
        if ticket is None:
            continue
        req = ticket.request
        try:
            front.set_state("generating", id=ticket.id)
            prompt = render_chat(tokenizer, req["messages"])
            room = engine.model.cos.size(0) - len(prompt)
            if room < 1:
                raise ValueError("the conversation does not fit the model's context")
            reply, shown = [], ""
            for column, _ in engine.generate(prompt, max_tokens=min(req["max_tokens"], room), temperature=req["temperature"],
                                             top_k=top_k, seed=req["seed"] % (2 ** 63), stop_tokens=(end,), top_p=req.get("top_p", 1.0)):
                if column[0] is None or column[0] == end:
                    continue
                reply.append(column[0])
                if req.get("stream"):
                    # a token may end inside a multi-byte character: only the text that is already stable goes out
                    text = tokenizer.decode(reply)
                    stable = text[:len(text) - 1] if text.endswith("\ufffd") else text
                    if len(stable) > len(shown) and stable.startswith(shown):
                        ticket.emit(stable[len(shown):])
                        shown = stable
            ticket.finish(text=tokenizer.decode(reply))
        except Exception as e:                                     # the front reports it as a 500 with this message
            ticket.finish(error=f"{type(e).__name__}: {e}")
        served += 1
        front.set_state("serving")
    return served
