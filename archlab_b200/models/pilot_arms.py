"""Matched-control pilot arms on the dense Qwen3.5 backbone: A keeps global attention everywhere, B turns the pilot layers
into local-window attention over the long window, C turns them into 2-simplicial attention over (short, long) windows.

What makes the three arms comparable (the reference's pilot, src/archlab/megatron/simplicial_attention.py:20-122 and
simplicial_pilot.py:250-310):

* all arms start from the *same* weights: the model is built once from one seed with global attention in every layer,
  and only then are the pilot layers re-armed; ``parameter_hashes(model, common_only=True)`` hashes the actual parameter
  bytes so a launcher can refuse arms whose shared weights differ;
* arm C's extra projections (second key / value per KV head and the second key norm) are drawn from a generator seeded
  by ``seed + 100000 + layer`` inside a forked RNG scope, so installing them does not move the global RNG stream that
  data order and dropout depend on, and the extra parameter count is known in closed form;
* arms B and C use the same long window, so C's only extra freedom is the short-window second key.
"""
from __future__ import annotations

import hashlib

import torch
import torch.nn as nn

from ..ops import simplicial as sx
from ..ops.attention import causal_attention
from .blocks import RMSNorm, apply_rope
from .qwen35 import DenseAttention, Qwen35Config, Qwen35LM

ARMS = ("A", "B", "C")
EXTRA_MARKERS = (".attn.k2.", ".attn.v2.", ".attn.k2_norm.")


def pilot_layers(n_layer: int, every: int = 4) -> tuple[int, ...]:
    """Layers ``every - 1, 2 * every - 1, ...`` (the last layer of every group), as in the 4B configuration."""
    return tuple(range(every - 1, n_layer, every))


class PilotAttention(nn.Module):
    """Re-armed attention of one pilot layer; shares the source layer's projections and norms."""

    def __init__(self, source: DenseAttention, arm: str, layer: int, *, short_window: int, long_window: int, seed: int):
        super().__init__()
        if arm not in ("B", "C"):
            raise ValueError("only arms B and C replace the attention core")
        if source.simplicial:
            raise ValueError("pilot arms start from a global-attention layer")
        c = self.c = source.c
        self.arm, self.short_window, self.long_window = arm, short_window, long_window
        self.qkv, self.o, self.q_norm, self.k_norm = source.qkv, source.o, source.q_norm, source.k_norm
        if arm == "C":
            kv = c.n_kv_heads * c.head_dim
            ref = source.qkv.weight
            devices = [ref.device.index] if ref.device.type == "cuda" else []
            with torch.random.fork_rng(devices=devices):              # the caller's RNG stream does not move
                torch.manual_seed(seed + 100_000 + layer)
                self.k2 = nn.Linear(c.hidden_size, kv, bias=False, device=ref.device, dtype=ref.dtype)
                self.v2 = nn.Linear(c.hidden_size, kv, bias=False, device=ref.device, dtype=ref.dtype)
                nn.init.normal_(self.k2.weight, std=0.02)
                nn.init.normal_(self.v2.weight, std=0.02)
            self.k2_norm = RMSNorm(c.head_dim, c.rms_eps).to(ref.device)
            self.k2_norm.load_state_dict(source.k_norm.state_dict())

    def forward(self, x, cos, sin):
        c = self.c
        B, T, _ = x.shape
        q_w, kv_w = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
        q, k1, v1 = self.qkv(x).split([q_w, kv_w, kv_w], -1)
        q = apply_rope(self.q_norm(q.view(B, T, c.n_heads, c.head_dim)), cos, sin)
        k1 = apply_rope(self.k_norm(k1.view(B, T, c.n_kv_heads, c.head_dim)), cos, sin)
        v1 = v1.view(B, T, c.n_kv_heads, c.head_dim)
        if self.arm == "B":
            o = causal_attention(q, k1, v1, window=self.long_window - 1)          # the query and long_window - 1 keys before it
        else:
            k2 = apply_rope(self.k2_norm(self.k2(x).view(B, T, c.n_kv_heads, c.head_dim)), cos, sin)
            v2 = self.v2(x).view(B, T, c.n_kv_heads, c.head_dim)
            o = sx.simplicial_attention(q, k1, k2, v1, v2, self.short_window, self.long_window)
        return self.o(o.reshape(B, T, q_w).to(x.dtype))


def extra_parameters(config: Qwen35Config, layers) -> int:
    """Parameters arm C adds: two KV-wide projections and one head-wide norm gain per pilot layer."""
    kv = config.n_kv_heads * config.head_dim
    return len(tuple(layers)) * (2 * config.hidden_size * kv + config.head_dim)


def build_arm(config: Qwen35Config, arm: str, *, seed: int = 42, layers=None, short_window: int = 16, long_window: int = 128,
              device=None) -> Qwen35LM:
    """The arm's model: one seeded global-attention initialisation shared by all arms, then the pilot layers re-armed."""
    if arm not in ARMS:
        raise ValueError("unknown pilot arm")
    if short_window < 1 or long_window < short_window:
        raise ValueError("windows must satisfy 1 <= short <= long")
    base = Qwen35Config(**{**config.to_dict(), "simplicial_every": 0})
    torch.manual_seed(seed)
    model = Qwen35LM(base)
    model.init_weights()
    if device is not None:
        model.to(device)
    layers = pilot_layers(base.n_layer) if layers is None else tuple(layers)
    if arm != "A":
        for i in layers:
            block = model.layers[i]
            block.attn = PilotAttention(block.attn, arm, i, short_window=short_window, long_window=long_window, seed=seed)
            block.layer_type = "local_attention" if arm == "B" else "simplicial_attention"
    model.pilot = {"arm": arm, "layers": list(layers), "short_window": short_window, "long_window": long_window, "seed": seed,
                   "extra_parameters": extra_parameters(base, layers) if arm == "C" else 0}
    return model


def parameter_hashes(model: nn.Module, *, common_only: bool = False) -> dict[str, str]:
    """SHA-256 of the actual parameter bytes per name (not of seeds or labels); ``common_only`` leaves out arm C's extras."""
    out = {}
    for name, p in model.named_parameters():
        if common_only and any(marker in f".{name}" for marker in EXTRA_MARKERS):
            continue
        out[name] = hashlib.sha256(p.detach().contiguous().view(torch.uint8).cpu().numpy().tobytes()).hexdigest()
    return out


def assert_matched(models: dict[str, nn.Module]) -> str:
    """All arms share the same common weights; returns the digest of the common set."""
    digests = {}
    for arm, model in models.items():
        hashes = parameter_hashes(model, common_only=True)
        digests[arm] = hashlib.sha256("".join(f"{k}:{v};" for k, v in sorted(hashes.items())).encode()).hexdigest()
    if len(set(digests.values())) != 1:
        raise ValueError(f"pilot arms do not share their common weights: {digests}")
    return next(iter(digests.values()))
