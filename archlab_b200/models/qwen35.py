"""Qwen3.5-style dense backbone and the ways 2-simplicial attention enters it.

* ``Qwen35LM``: dense GQA + SwiGLU decoder (4B geometry: 36 layers, hidden 2560, 32 Q / 8 KV heads of
  128, FFN 9728, vocab 151936) where every ``simplicial_every``-th layer's attention is the
  2-simplicial operator (window w2 x w1) instead of softmax attention.
* ``InsertedBranch`` / ``install``: additive pre-norm attention branches (mechanism ``simplicial`` or
  the parameter-matched ``local`` control) attached AFTER chosen decoder layers of ANY model with a
  ``.layers`` list through forward hooks; zero-initialised output projection, sigmoid output gate;
  ``stratified_sites`` picks the same fraction of every layer type; ``freeze_backbone`` trains the
  branches only (src/archlab/architectures/qwen35_insertion.py:32-176).
* ``SimplicialSwitch``: replaces a full-attention layer by the full-causal determinant simplicial
  form with SO(3) chunk rotary embedding, inheriting the teacher's q/k/v/o and adding k2 / v2
  (src/archlab/architectures/qwen35_switch.py:41-218).
"""
from __future__ import annotations

from dataclasses import asdict, dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import block_ops
from ..ops import local_attention as la
from ..ops.attention import causal_attention
from ..ops import simplicial as sx
from .blocks import GroupRMSNorm, RMSNorm, apply_rope, rope_tables, so3_chunk_rope


# ------------------------------------------------------------------------------------------------
# dense backbone
# ------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class Qwen35Config:
    vocab_size: int = 151_936
    sequence_len: int = 8192
    n_layer: int = 36
    hidden_size: int = 2560
    n_heads: int = 32
    n_kv_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 9728
    rope_theta: float = 1e6
    rms_eps: float = 1e-6
    simplicial_every: int = 4           # 0: none; k: layers k-1, 2k-1, ... use 2-simplicial attention
    simplicial_w1: int = 32
    simplicial_w2: int = 512
    tie_embeddings: bool = False

    @classmethod
    def tiny(cls, **kw):
        base = dict(vocab_size=256, sequence_len=64, n_layer=4, hidden_size=64, n_heads=4, n_kv_heads=2, head_dim=16,
                    intermediate_size=128, simplicial_every=2, simplicial_w1=4, simplicial_w2=8)
        base.update(kw)
        return cls(**base)

    def is_simplicial(self, layer: int) -> bool:
        return self.simplicial_every > 0 and (layer + 1) % self.simplicial_every == 0

    def to_dict(self):
        return asdict(self)


def _lin(i, o):
    return nn.Linear(i, o, bias=False)


class DenseAttention(nn.Module):
    def __init__(self, c: Qwen35Config, simplicial: bool):
        super().__init__()
        self.c, self.simplicial = c, simplicial
        q, kv = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
        self.qkv = _lin(c.hidden_size, q + (4 if simplicial else 2) * kv)      # q, k1, v1 (, k2, v2)
        self.o = _lin(q, c.hidden_size)
        self.q_norm, self.k_norm = RMSNorm(c.head_dim, c.rms_eps), RMSNorm(c.head_dim, c.rms_eps)
        if simplicial:
            self.k2_norm = RMSNorm(c.head_dim, c.rms_eps)

    def forward(self, x, cos, sin):
        c = self.c
        B, T, _ = x.shape
        q_w, kv_w = c.n_heads * c.head_dim, c.n_kv_heads * c.head_dim
        parts = self.qkv(x).split([q_w] + [kv_w] * (4 if self.simplicial else 2), -1)
        q = apply_rope(self.q_norm(parts[0].view(B, T, c.n_heads, c.head_dim)), cos, sin)
        kv = [p.view(B, T, c.n_kv_heads, c.head_dim) for p in parts[1:]]
        k1 = apply_rope(self.k_norm(kv[0]), cos, sin)
        if self.simplicial:
            k2 = apply_rope(self.k2_norm(kv[2]), cos, sin)
            o = sx.simplicial_attention(q, k1, k2, kv[1], kv[3], c.simplicial_w1, c.simplicial_w2)
        else:
            o = causal_attention(q, k1, kv[1])
        return self.o(o.reshape(B, T, q_w).to(x.dtype))


class DenseBlock(nn.Module):
    def __init__(self, c: Qwen35Config, layer: int):
        super().__init__()
        self.layer_type = "simplicial_attention" if c.is_simplicial(layer) else "full_attention"
        self.input_norm, self.post_norm = RMSNorm(c.hidden_size, c.rms_eps), RMSNorm(c.hidden_size, c.rms_eps)
        self.attn = DenseAttention(c, c.is_simplicial(layer))
        self.gate_up = _lin(c.hidden_size, 2 * c.intermediate_size)
        self.down = _lin(c.intermediate_size, c.hidden_size)

    def forward(self, x, cos=None, sin=None, **_):
        x = x + self.attn(self.input_norm(x), cos, sin)
        return x + self.down(block_ops.swiglu(self.gate_up(self.post_norm(x))))


class Qwen35LM(nn.Module):
    def __init__(self, config: Qwen35Config):
        super().__init__()
        c = self.config = config
        self.embed = nn.Embedding(c.vocab_size, c.hidden_size)
        self.layers = nn.ModuleList(DenseBlock(c, i) for i in range(c.n_layer))
        self.norm = RMSNorm(c.hidden_size, c.rms_eps)
        self.lm_head = _lin(c.hidden_size, c.vocab_size)
        if c.tie_embeddings:
            self.lm_head.weight = self.embed.weight

    @torch.no_grad()
    def init_weights(self, std: float = 0.02):
        for _, p in self.named_parameters():
            if p.ndim >= 2:
                nn.init.normal_(p, std=std)
        for m in self.modules():                     # gains and biases too: a meta-built model has no defaults
            if isinstance(m, RMSNorm):
                m.weight.fill_(0.0 if m.zero_centered else 1.0)
            elif isinstance(m, nn.Linear) and m.bias is not None:
                m.bias.zero_()

    def layer_types(self) -> list[str]:
        return [b.layer_type for b in self.layers]

    def parameter_count(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def forward(self, ids, labels=None):
        c = self.config
        B, T = ids.shape
        dt = torch.bfloat16 if ids.device.type == "cuda" else torch.float32
        x = self.embed(ids).to(dt)
        cos, sin = rope_tables(T, c.head_dim, c.rope_theta, ids.device)
        with torch.autocast(ids.device.type, dtype=dt, enabled=dt != torch.float32):
            for blk in self.layers:
                x = blk(x, cos=cos, sin=sin)
            logits = self.lm_head(self.norm(x))
        if labels is None:
            return logits.float()
        flat = labels.flatten()
        return block_ops.cross_entropy_sum(logits.flatten(0, 1), flat) / flat.ne(-1).sum().clamp_min(1)


# ------------------------------------------------------------------------------------------------
# additive branches inserted after chosen layers
# ------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class InsertionConfig:
    hidden_size: int
    mechanism: str = "simplicial"
    query_heads: int = 16
    kv_heads: int = 4
    head_dim: int = 256
    short_window: int = 16
    long_window: int = 128
    rotary_fraction: float = 0.25
    rope_theta: float = 1e7
    rms_norm_eps: float = 1e-6
    initializer_std: float = 0.02
    output_initialization: str = "zeros"

    def __post_init__(self):
        if self.mechanism not in ("simplicial", "local"):
            raise ValueError("mechanism must be simplicial or local")
        if self.query_heads % self.kv_heads or min(self.query_heads, self.kv_heads, self.head_dim) < 1:
            raise ValueError("KV heads must divide query heads")
        if not 1 <= self.short_window <= self.long_window:
            raise ValueError("windows must satisfy 1 <= short <= long")
        rot = int(self.head_dim * self.rotary_fraction)
        if rot < 2 or rot % 2:
            raise ValueError("partial RoPE must keep a positive even dimension")
        if self.output_initialization not in ("zeros", "normal"):
            raise ValueError("output initialization must be zeros or normal")

    def branch_parameters(self) -> int:
        q, kv = self.query_heads * self.head_dim, self.kv_heads * self.head_dim
        streams = 2 if self.mechanism == "simplicial" else 1
        return self.hidden_size * (3 * q + 2 * streams * kv) + self.hidden_size + (1 + streams) * self.head_dim


class InsertedBranch(nn.Module):
    def __init__(self, config: InsertionConfig, *, seed: int, backend: str = "kernel"):
        super().__init__()
        c = self.config = config
        self.backend = backend
        streams = 2 if c.mechanism == "simplicial" else 1
        W, q, kv = c.hidden_size, c.query_heads * c.head_dim, c.kv_heads * c.head_dim
        with torch.random.fork_rng(devices=[]):
            torch.manual_seed(seed)
            self.norm = GroupRMSNorm(W, 1, c.rms_norm_eps, zero_centered=True)
            self.q, self.output_gate = _lin(W, q), _lin(W, q)
            self.keys = nn.ModuleList(_lin(W, kv) for _ in range(streams))
            self.values = nn.ModuleList(_lin(W, kv) for _ in range(streams))
            self.output = _lin(q, W)
            self.q_norm = GroupRMSNorm(c.head_dim, 1, c.rms_norm_eps, zero_centered=True)
            self.k_norms = nn.ModuleList(GroupRMSNorm(c.head_dim, 1, c.rms_norm_eps, zero_centered=True) for _ in range(streams))
            for m in self.modules():
                if isinstance(m, nn.Linear):
                    nn.init.normal_(m.weight, std=c.initializer_std)
            if c.output_initialization == "zeros":
                nn.init.zeros_(self.output.weight)

    def forward(self, hidden: torch.Tensor, position_ids: torch.Tensor | None = None) -> torch.Tensor:
        c = self.config
        B, T, _ = hidden.shape
        rot = int(c.head_dim * c.rotary_fraction)
        cos, sin = rope_tables(T, rot, c.rope_theta, hidden.device)
        x = self.norm(hidden)
        q = apply_rope(self.q_norm(self.q(x).view(B, T, c.query_heads, c.head_dim)), cos, sin, rot_dim=rot)
        ks = [apply_rope(n(k(x).view(B, T, c.kv_heads, c.head_dim)), cos, sin, rot_dim=rot)
              for k, n in zip(self.keys, self.k_norms)]
        vs = [v(x).view(B, T, c.kv_heads, c.head_dim) for v in self.values]
        if c.mechanism == "simplicial":
            core = sx.simplicial_attention if self.backend == "kernel" else sx.simplicial_attention_reference
            att = core(q, ks[0], ks[1], vs[0], vs[1], c.short_window, c.long_window)
        else:
            core = la.local_attention if self.backend == "kernel" else la.reference_local_attention
            att = core(q, ks[0], vs[0], c.long_window)
        gated = att.flatten(-2).float() * torch.sigmoid(self.output_gate(x).float())
        return self.output(gated.to(hidden.dtype))


def stratified_sites(layer_types: list[str], fraction: float = 0.25) -> list[int]:
    """The same ``fraction`` of each layer type, evenly spaced within the type."""
    if not 0 < fraction <= 1:
        raise ValueError("fraction must be in (0, 1]")
    sites = []
    for kind in sorted(set(layer_types)):
        idx = [i for i, t in enumerate(layer_types) if t == kind]
        n = max(1, round(len(idx) * fraction))
        stride = len(idx) / n
        sites += [idx[int((j + 1) * stride) - 1] for j in range(n)]
    return sorted(sites)


def decoder_layers(model: nn.Module) -> nn.ModuleList:
    inner = getattr(model, "model", model)
    inner = getattr(inner, "language_model", inner)
    return inner.layers


def install(model: nn.Module, config: InsertionConfig, sites: list[int], *, seed: int = 42, backend: str = "kernel") -> list:
    """Attach one branch after each site layer; returns the hook handles (``remove()`` detaches)."""
    if hasattr(model, "inserted_branches"):
        raise ValueError("branches are already installed")
    layers = decoder_layers(model)
    if not sites or any(not 0 <= s < len(layers) for s in sites) or len(set(sites)) != len(sites):
        raise ValueError("sites must be distinct decoder-layer indices")
    ref = next(model.parameters())
    branches = nn.ModuleDict({str(s): InsertedBranch(config, seed=seed + s, backend=backend) for s in sites})
    model.inserted_branches = branches.to(device=ref.device, dtype=ref.dtype)
    model.inserted_sites = list(sites)

    def hook(module, args, kwargs, output):
        hidden = output[0] if isinstance(output, tuple) else output
        updated = hidden + model.inserted_branches[str(module.archlab_site)](hidden, kwargs.get("position_ids"))
        return (updated, *output[1:]) if isinstance(output, tuple) else updated

    handles = []
    for s in sites:
        layers[s].archlab_site = s
        handles.append(layers[s].register_forward_hook(hook, with_kwargs=True))
    return handles


def freeze_backbone(model: nn.Module) -> dict:
    trainable = frozen = 0
    for name, p in model.named_parameters():
        p.requires_grad_(name.startswith("inserted_branches."))
        trainable += p.numel() if p.requires_grad else 0
        frozen += 0 if p.requires_grad else p.numel()
    return {"trainable": trainable, "frozen": frozen}


def describe(config: InsertionConfig, sites: list[int], layer_types: list[str]) -> dict:
    return {"config": asdict(config), "sites": sites, "site_types": [layer_types[s] for s in sites],
            "branch_parameters": config.branch_parameters() * len(sites)}


# ------------------------------------------------------------------------------------------------
# switch: replace a softmax-attention layer by the determinant simplicial form
# ------------------------------------------------------------------------------------------------
class SimplicialSwitch(nn.Module):
    """Full-causal determinant 2-simplicial attention that starts as a copy of a teacher attention
    layer: q / k / v / o weights are inherited, the second key / value streams are new (zero weights,
    bias 1, so the product reduces to the teacher's operands at initialisation)."""

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, *, max_window: int = 1 << 30):
        super().__init__()
        if head_dim % 3:
            raise ValueError("determinant scores need head_dim to be a multiple of 3")
        self.h, self.kv, self.d, self.window = n_heads, n_kv_heads, head_dim, max_window
        self.q, self.k, self.v = _lin(hidden, n_heads * head_dim), _lin(hidden, n_kv_heads * head_dim), _lin(hidden, n_kv_heads * head_dim)
        self.k2 = nn.Linear(hidden, n_kv_heads * head_dim, bias=True)
        self.v2 = nn.Linear(hidden, n_kv_heads * head_dim, bias=True)
        self.o = _lin(n_heads * head_dim, hidden)
        with torch.no_grad():
            for m in (self.k2, self.v2):
                m.weight.zero_()
                m.bias.fill_(1.0)

    @torch.no_grad()
    def inherit(self, q_w, k_w, v_w, o_w):
        for dst, src in ((self.q, q_w), (self.k, k_w), (self.v, v_w), (self.o, o_w)):
            dst.weight.copy_(src)

    def forward(self, x):
        B, T, _ = x.shape
        pos = torch.arange(T, device=x.device).view(1, T, 1)
        shp = lambda t, h: t.view(B, T, h, self.d)
        q = so3_chunk_rope(shp(self.q(x), self.h), pos)
        k1 = so3_chunk_rope(shp(self.k(x), self.kv), pos)
        k2 = so3_chunk_rope(shp(self.k2(x), self.kv), pos)
        w = min(T, self.window)
        o = sx.determinant_simplicial_attention(q, k1, k2, shp(self.v(x), self.kv), shp(self.v2(x), self.kv), w, w)
        return self.o(o.reshape(B, T, self.h * self.d).to(x.dtype))
