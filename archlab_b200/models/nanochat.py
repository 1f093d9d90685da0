"""nanochat-style speedrun GPT: the plain PyTorch definition.

This module is the *semantic* definition of the flagship model (parameter names, init, forward
arithmetic) and the execution path on CPU / gloo.  On a B200 the same parameters are driven by
``archlab_b200.models.nanochat_engine.FusedGPTEngine``, which runs hand-written sm_100a kernels
and is checked against this module in the GPU tests.

Behaviour follows the reference's ``GPT`` (src/archlab/architectures/base.py:103-143 config,
:231-265 QK features, :268-353 attention, :356-366 ReLU^2 MLP, :566-683 init, :864-1012 forward):
RoPE base 1e5 half-split, parameter-free RMSNorm, QK-norm x1.2, untied wte / lm_head, value
embeddings on alternating layers with a 12-channel sigmoid gate x3, per-layer resid / x0 lambdas,
smear gate, mid-layer backout, 15*tanh logit soft-cap, sliding-window pattern "SSSL".
A layer listed in ``simplicial_layers`` swaps its attention for 2-simplicial attention
(``archlab_b200.ops.simplicial``) with windows ``simplicial_w1`` x ``simplicial_w2``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class GPTConfig:
    sequence_len: int = 2048
    vocab_size: int = 32768
    n_layer: int = 12
    n_head: int = 6
    n_kv_head: int = 6
    n_embd: int = 768
    window_pattern: str = "SSSL"
    rope_fraction: float = 1.0
    embedding_init_std: float = 0.8
    matrix_init_recipe: str = "speedrun-zero-proj"
    logit_softcap: float = 15.0
    z_loss_weight: float = 0.0
    mlp_ratio: int = 4
    value_embeddings: bool = True
    simplicial_layers: tuple[int, ...] = ()
    simplicial_w1: int = 16     # short window (k1 / v1)
    simplicial_w2: int = 64     # long window (k2 / v2)
    compute_dtype: torch.dtype = torch.float32

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head

    @property
    def padded_vocab(self) -> int:
        return (self.vocab_size + 63) // 64 * 64

    @classmethod
    def from_depth(cls, depth: int, *, aspect_ratio: int = 64, head_dim: int = 128, **kw) -> "GPTConfig":
        """The speedrun sizing rule: d_model = depth * aspect_ratio rounded up to a multiple of
        head_dim (src/archlab/speedrun/base_train.py:442-445): depth 20 -> 1280 wide, 10 heads."""
        base = depth * aspect_ratio
        n_embd = (base + head_dim - 1) // head_dim * head_dim
        n_head = n_embd // head_dim
        return cls(n_layer=depth, n_embd=n_embd, n_head=n_head, n_kv_head=n_head, **kw)


def rms_norm(x: torch.Tensor) -> torch.Tensor:
    return F.rms_norm(x, (x.size(-1),))


def has_ve(layer_idx: int, n_layer: int) -> bool:
    return layer_idx % 2 == (n_layer - 1) % 2


def window_sizes(config: GPTConfig) -> list[int]:
    """Left-window per layer (keys i-left..i are visible); the last layer is always full."""
    long_w = config.sequence_len
    short_w = -(-long_w // 4 // 128) * 128
    table = {"L": long_w, "S": short_w}
    pattern = config.window_pattern.upper()
    if not pattern or any(c not in "SL" for c in pattern):
        raise ValueError(f"invalid window_pattern {config.window_pattern!r}")
    out = [table[pattern[i % len(pattern)]] for i in range(config.n_layer)]
    out[-1] = long_w
    return out


def rotary_tables(seq_len: int, head_dim: int, dtype: torch.dtype, device=None, base: float = 100000.0):
    ch = torch.arange(0, head_dim, 2, dtype=torch.float32, device=device)
    inv = 1.0 / (base ** (ch / head_dim))
    t = torch.arange(seq_len, dtype=torch.float32, device=device)
    fr = torch.outer(t, inv)
    return fr.cos().to(dtype), fr.sin().to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, T, H, D]; cos/sin [T, D/2]; half-split rotation."""
    d = x.size(-1) // 2
    c, s = cos[None, :, None, :], sin[None, :, None, :]
    x1, x2 = x[..., :d], x[..., d:]
    return torch.cat([x1 * c + x2 * s, x1 * (-s) + x2 * c], dim=-1)


def sdpa_window(q, k, v, window: int) -> torch.Tensor:
    """q [B,T,Hq,D], k/v [B,T,Hkv,D] -> [B,T,Hq,D]; causal with a left window (−1 = unlimited)."""
    T = q.size(1)
    q, k, v = (t.transpose(1, 2) for t in (q, k, v))
    gqa = q.size(1) != k.size(1)
    if window < 0 or window >= T:
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=gqa)
    else:
        i = torch.arange(T, device=q.device).view(T, 1)
        j = torch.arange(T, device=q.device).view(1, T)
        mask = (j <= i) & ((i - j) <= window)
        y = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, enable_gqa=gqa)
    return y.transpose(1, 2)


class CastLinear(nn.Linear):
    """fp32 master weight, matmul in the activation dtype."""

    def __init__(self, i: int, o: int):
        super().__init__(i, o, bias=False)

    def forward(self, x):
        return F.linear(x, self.weight.to(x.dtype))


class CausalSelfAttention(nn.Module):
    def __init__(self, config: GPTConfig, layer_idx: int):
        super().__init__()
        self.config, self.layer_idx = config, layer_idx
        C, H, Hkv, D = config.n_embd, config.n_head, config.n_kv_head, config.head_dim
        self.c_q = CastLinear(C, H * D)
        self.c_k = CastLinear(C, Hkv * D)
        self.c_v = CastLinear(C, Hkv * D)
        self.c_proj = CastLinear(C, C)
        self.ve_gate_channels = min(12, C)
        use_ve = config.value_embeddings and has_ve(layer_idx, config.n_layer)
        self.ve_gate = CastLinear(self.ve_gate_channels, Hkv) if use_ve else None

    def forward(self, x, ve, cos, sin, window):
        B, T, _ = x.shape
        cfg = self.config
        q = self.c_q(x).view(B, T, cfg.n_head, cfg.head_dim)
        k = self.c_k(x).view(B, T, cfg.n_kv_head, cfg.head_dim)
        v = self.c_v(x).view(B, T, cfg.n_kv_head, cfg.head_dim)
        if ve is not None:
            gate = 3 * torch.sigmoid(self.ve_gate(x[..., : self.ve_gate_channels]))
            v = v + gate.unsqueeze(-1) * ve.view_as(v)
        q = rms_norm(apply_rope(q, cos, sin)) * 1.2
        k = rms_norm(apply_rope(k, cos, sin)) * 1.2
        y = sdpa_window(q, k, v, window)
        return self.c_proj(y.contiguous().view(B, T, -1))


class MLP(nn.Module):
    def __init__(self, config: GPTConfig):
        super().__init__()
        self.c_fc = CastLinear(config.n_embd, config.mlp_ratio * config.n_embd)
        self.c_proj = CastLinear(config.mlp_ratio * config.n_embd, config.n_embd)

    def forward(self, x):
        return self.c_proj(F.relu(self.c_fc(x)).square())


class Block(nn.Module):
    def __init__(self, config: GPTConfig, layer_idx: int):
        super().__init__()
        if layer_idx in config.simplicial_layers:
            from .simplicial_layer import SimplicialSelfAttention

            self.attn = SimplicialSelfAttention(config, layer_idx)
        else:
            self.attn = CausalSelfAttention(config, layer_idx)
        self.mlp = MLP(config)

    def forward(self, x, ve, cos, sin, window):
        x = x + self.attn(rms_norm(x), ve, cos, sin, window)
        return x + self.mlp(rms_norm(x))


class GPT(nn.Module):
    """Parameter container + eager forward.  Construct on the meta device and call
    ``init_weights()`` after ``to_empty`` (or construct directly on a real device)."""

    def __init__(self, config: GPTConfig):
        super().__init__()
        self.config = config
        C, V = config.n_embd, config.padded_vocab
        self.window_sizes = window_sizes(config)
        self.transformer = nn.ModuleDict({
            "wte": nn.Embedding(V, C),
            "h": nn.ModuleList([Block(config, i) for i in range(config.n_layer)]),
        })
        self.lm_head = CastLinear(C, V)
        self.resid_lambdas = nn.Parameter(torch.ones(config.n_layer))
        self.x0_lambdas = nn.Parameter(torch.zeros(config.n_layer))
        self.smear_gate_channels = min(24, C)
        self.smear_gate = CastLinear(self.smear_gate_channels, 1)
        self.smear_lambda = nn.Parameter(torch.zeros(1))
        self.backout_lambda = nn.Parameter(0.2 * torch.ones(1))
        kv_dim = config.n_kv_head * config.head_dim
        self.value_embeds = nn.ModuleDict({
            str(i): nn.Embedding(V, kv_dim)
            for i in range(config.n_layer)
            if config.value_embeddings and has_ve(i, config.n_layer)
            and i not in config.simplicial_layers
        })
        self.rotary_seq_len = config.sequence_len
        cos, sin = rotary_tables(self.rotary_seq_len, config.head_dim, config.compute_dtype, device="cpu")
        self.register_buffer("cos", cos, persistent=False)
        self.register_buffer("sin", sin, persistent=False)

    # -------------------------------------------------------------------------------- init
    @torch.no_grad()
    def init_weights(self) -> None:
        cfg = self.config
        nn.init.normal_(self.transformer.wte.weight, mean=0.0, std=cfg.embedding_init_std)
        nn.init.normal_(self.lm_head.weight, mean=0.0, std=0.001)
        s = 3 ** 0.5 * cfg.n_embd ** -0.5
        for block in self.transformer.h:
            attn = block.attn
            for name in ("c_q", "c_k", "c_v", "c_k2", "c_v2"):
                if hasattr(attn, name):
                    nn.init.uniform_(getattr(attn, name).weight, -s, s)
            if cfg.matrix_init_recipe == "speedrun-zero-proj":
                nn.init.zeros_(attn.c_proj.weight)
                nn.init.uniform_(block.mlp.c_fc.weight, -0.4 * s, 0.4 * s)
                nn.init.zeros_(block.mlp.c_proj.weight)
            elif cfg.matrix_init_recipe == "hyperball":
                nn.init.normal_(attn.c_proj.weight, std=0.72 * cfg.n_embd ** -0.5)
                nn.init.normal_(block.mlp.c_fc.weight, std=0.86 * cfg.n_embd ** -0.5)
                nn.init.normal_(block.mlp.c_proj.weight, std=0.86 * cfg.n_embd ** -0.5)
            elif cfg.matrix_init_recipe == "normal-0.02":
                # random-init benchmark recipe: every matrix N(0, 0.02)
                for w in (attn.c_proj.weight, block.mlp.c_fc.weight, block.mlp.c_proj.weight):
                    nn.init.normal_(w, std=0.02)
            else:
                raise ValueError(f"unknown matrix_init_recipe={cfg.matrix_init_recipe!r}")
        n = cfg.n_layer
        for i in range(n):
            self.resid_lambdas[i] = 1.15 - 0.10 * i / max(n - 1, 1)
            self.x0_lambdas[i] = 0.20 - 0.15 * i / max(n - 1, 1)
        for ve in self.value_embeds.values():
            nn.init.uniform_(ve.weight, -s, s)
        for block in self.transformer.h:
            if getattr(block.attn, "ve_gate", None) is not None:
                nn.init.uniform_(block.attn.ve_gate.weight, 0.0, 0.02)
        nn.init.uniform_(self.smear_gate.weight, 0.0, 0.02)
        self.smear_lambda.zero_()
        self.backout_lambda.fill_(0.2)
        dev = self.transformer.wte.weight.device
        cos, sin = rotary_tables(self.rotary_seq_len, cfg.head_dim, cfg.compute_dtype, device=dev)
        self.cos, self.sin = cos, sin

    # -------------------------------------------------------------------------------- metadata
    def estimate_flops(self) -> int:
        """FLOPs per token, forward + backward: 6 per matmul parameter plus 12*h*d*effective
        context per layer (src/archlab/architectures/base.py:755-799)."""
        cfg = self.config
        nparams = sum(p.numel() for p in self.parameters())
        exclude = self.transformer.wte.weight.numel()
        exclude += sum(ve.weight.numel() for ve in self.value_embeds.values())
        exclude += self.resid_lambdas.numel() + self.x0_lambdas.numel()
        exclude += self.smear_gate.weight.numel() + self.smear_lambda.numel() + self.backout_lambda.numel()
        attn = sum(12 * cfg.n_head * cfg.head_dim * min(w, cfg.sequence_len) for w in self.window_sizes)
        return 6 * (nparams - exclude) + attn

    def num_scaling_params(self) -> dict[str, int]:
        wte = self.transformer.wte.weight.numel()
        ve = sum(v.weight.numel() for v in self.value_embeds.values())
        head = self.lm_head.weight.numel()
        blocks = sum(p.numel() for p in self.transformer.h.parameters())
        scalars = (self.resid_lambdas.numel() + self.x0_lambdas.numel() + self.smear_gate.weight.numel()
                   + self.smear_lambda.numel() + self.backout_lambda.numel())
        out = {"wte": wte, "value_embeds": ve, "lm_head": head, "transformer_matrices": blocks,
               "scalars": scalars}
        out["total"] = sum(out.values())
        assert out["total"] == sum(p.numel() for p in self.parameters())
        return out

    # -------------------------------------------------------------------------------- forward
    def embed(self, idx: torch.Tensor) -> torch.Tensor:
        cfg = self.config
        x = rms_norm(self.transformer.wte(idx).to(cfg.compute_dtype))
        G = self.smear_gate_channels
        gate = self.smear_lambda.to(x.dtype) * torch.sigmoid(self.smear_gate(x[:, 1:, :G]))
        return torch.cat([x[:, :1], x[:, 1:] + gate * x[:, :-1]], dim=1)

    def trunk(self, idx: torch.Tensor) -> torch.Tensor:
        cfg = self.config
        T = idx.size(1)
        cos, sin = self.cos[:T], self.sin[:T]
        x = self.embed(idx)
        x0 = x
        x_backout = None
        for i, block in enumerate(self.transformer.h):
            x = self.resid_lambdas[i].to(x.dtype) * x + self.x0_lambdas[i].to(x.dtype) * x0
            ve = self.value_embeds[str(i)](idx).to(x.dtype) if str(i) in self.value_embeds else None
            x = block(x, ve, cos, sin, self.window_sizes[i])
            if i == cfg.n_layer // 2:
                x_backout = x
        if x_backout is not None:
            x = x - self.backout_lambda.to(x.dtype) * x_backout
        return rms_norm(x)

    def forward(self, idx, targets=None, loss_reduction: str = "mean"):
        cfg = self.config
        x = self.trunk(idx)
        raw = self.lm_head(x)[..., : cfg.vocab_size]
        logits = raw.float()
        logits = cfg.logit_softcap * torch.tanh(logits / cfg.logit_softcap)
        if targets is None:
            return logits
        loss = F.cross_entropy(logits.reshape(-1, logits.size(-1)), targets.reshape(-1),
                               ignore_index=-1, reduction=loss_reduction)
        if self.training and cfg.z_loss_weight > 0:
            valid = targets.ne(-1)
            z = torch.logsumexp(raw.float(), dim=-1).square()
            z = torch.where(valid, z, torch.zeros_like(z))
            if loss_reduction == "none":
                z = z.reshape(-1)
            elif loss_reduction == "sum":
                z = z.sum()
            else:
                z = z.sum() / valid.sum().clamp_min(1)
            loss = loss + cfg.z_loss_weight * z
        return loss

    @torch.inference_mode()
    def generate(self, tokens: list[int], max_tokens: int, temperature: float = 1.0, top_k=None, seed=42):
        """Naive (no KV cache) autoregressive sampling; yields one token id at a time."""
        dev = self.transformer.wte.weight.device
        rng = torch.Generator(device=dev).manual_seed(seed) if temperature > 0 else None
        ids = torch.tensor([tokens], dtype=torch.long, device=dev)
        for _ in range(max_tokens):
            logits = self.forward(ids[:, -self.config.sequence_len:])[:, -1, :]
            if top_k is not None and top_k > 0:
                v, _ = torch.topk(logits, min(top_k, logits.size(-1)))
                logits[logits < v[:, [-1]]] = -float("inf")
            if temperature > 0:
                nxt = torch.multinomial(F.softmax(logits / temperature, dim=-1), 1, generator=rng)
            else:
                nxt = torch.argmax(logits, dim=-1, keepdim=True)
            ids = torch.cat([ids, nxt], dim=1)
            yield int(nxt.item())


from .protocol import attach_protocol  # noqa: E402  (after the classes it completes)

attach_protocol(GPT)
