"""Long-context training replay of a Limite model: layer-wise recomputation, one shared execution context, attention whose
memory is linear in the sequence on every path.

At 131 072 tokens the activations of a 24-layer model do not fit if autograd keeps every layer's intermediates, and a
single [T, T] integer temporary is 128 GiB.  ``replay_hidden`` therefore

* runs every decoder layer under a non-reentrant checkpoint: only the layer inputs stay alive between forward and
  backward, the rest is rebuilt layer by layer;
* looks up positions and RoPE tables ONCE per geometry in a ``ReplayContextCache`` and hands the same tensors to every
  layer and every step; the cache can be locked, after which an unseen geometry raises instead of allocating (the state
  wanted before a CUDA-graph capture);
* reduces attention with the sm_100a flash kernel where it applies (bf16, head_dim 128: the window is a kernel
  argument, no mask exists at all) and otherwise with ``bounded_window_attention``: query tiles that see only the keys
  of their window, each tile under its own checkpoint so that rebuilding a layer does not keep all tiles' scores.
  Masks are boolean and tile-sized; the scalar window is subtracted before broadcasting.

``replay_loss`` adds the chunked vocabulary projection.  (The reference replays an external implementation of the model
the same way: src/archlab/architectures/limite_replay.py:57-135,209-222, limite_context.py:16-66.)
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
from torch.utils.checkpoint import checkpoint

from ..ops.attention import causal_attention, kernel_supports
from .blocks import rope_tables
from .limite import LimiteLM, chunked_logits_processor, logprob_entropy_processor


@dataclass(frozen=True)
class ReplayContext:
    key: tuple
    positions: torch.Tensor
    cos: torch.Tensor
    sin: torch.Tensor


def context_key(model: LimiteLM, ids: torch.Tensor, trainable_mode: str = "full") -> tuple:
    """Everything the execution tensors depend on, read without touching tensor values."""
    c = model.config
    return (tuple(ids.shape), ids.device.type, ids.device.index, model.embed.weight.dtype, model.training, trainable_mode,
            c.sliding_window, tuple(c.global_layers), c.head_dim, c.rope_theta)


class ReplayContextCache:
    """Holds one context (execution tensors only, never parameters); off until enabled."""

    def __init__(self):
        self.enabled, self.locked, self.entry, self.builds = False, False, None, 0

    def enable(self, enabled: bool = True) -> None:
        self.enabled = bool(enabled)
        if not enabled:
            self.entry, self.locked = None, False

    def invalidate(self) -> None:
        self.entry = None

    def lock(self, locked: bool = True) -> None:
        self.locked = bool(locked)

    def prepare(self, model: LimiteLM, ids: torch.Tensor, trainable_mode: str = "full") -> ReplayContext:
        if not self.enabled:
            raise RuntimeError("enable the replay context cache before preparing a context")
        key = context_key(model, ids, trainable_mode)
        if self.entry is not None and self.entry.key == key:
            return self.entry
        if self.locked or (ids.is_cuda and torch.cuda.is_current_stream_capturing()):
            raise RuntimeError("prepare the replay context before capture; the cache key changed")
        self.entry = _build_context(model, ids, key)
        self.builds += 1
        return self.entry


def _build_context(model, ids, key) -> ReplayContext:
    c = model.config
    cos, sin = rope_tables(ids.size(1), c.head_dim, c.rope_theta, ids.device)
    positions = torch.arange(ids.size(1), device=ids.device)[None].expand(ids.size(0), -1)
    return ReplayContext(key, positions, cos, sin)


def _tile(q, k, v, window, query_start, key_start):
    """Softmax attention of one query tile over its key span, fp32; positions are absolute."""
    D, g = q.shape[-1], q.shape[2] // k.shape[2]
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
    if g > 1:
        kf, vf = kf.repeat_interleave(g, 1), vf.repeat_interleave(g, 1)
    qi = torch.arange(query_start, query_start + q.shape[1], device=q.device)[:, None]
    kj = torch.arange(key_start, key_start + k.shape[1], device=q.device)[None, :]
    allowed = kj <= qi
    if window >= 0:
        allowed = allowed.logical_and_(kj >= qi - window)         # scalar first: no [tile, span] integer age tensor survives
    s = (qf @ kf.transpose(-1, -2) / math.sqrt(D)).masked_fill_(~allowed, float("-inf"))
    return (torch.softmax(s, -1) @ vf).transpose(1, 2).to(q.dtype)


def bounded_window_attention(q, k, v, window: int, *, query_tile: int = 1024) -> torch.Tensor:
    """q [B, T, Hq, D], k / v [B, T, Hkv, D]; ``window`` = keys before the query that it sees (-1: all).  Memory is
    O(query_tile x (query_tile + window)) per tile for local layers; each tile is recomputed on its own in backward."""
    T = q.shape[1]
    outs = []
    for start in range(0, T, query_tile):
        end = min(T, start + query_tile)
        key_start = 0 if window < 0 else max(0, start - window)
        args = (q[:, start:end], k[:, key_start:end], v[:, key_start:end], window, start, key_start)
        if torch.is_grad_enabled() and any(t.requires_grad for t in args[:3]):
            outs.append(checkpoint(_tile, *args, use_reentrant=False))
        else:
            outs.append(_tile(*args))
    return torch.cat(outs, 1)


def _reduce(attn, q, k, v, query_tile):
    if kernel_supports(q, k):
        return causal_attention(q, k, v, -1 if attn.is_global else attn.c.sliding_window)
    return bounded_window_attention(q, k, v, -1 if attn.is_global else attn.c.sliding_window, query_tile=query_tile)


def _layer(block, x, ve, cos, sin, query_tile):
    if block.prelude is not None:
        x = x + block.prelude(x, cos, sin)
    h = block.input_norm(x)
    q, k, v = block.attn.project(h, ve, cos, sin)
    x = x + block.attn.finish(h, _reduce(block.attn, q, k, v, query_tile))
    from ..ops import block_ops

    return x + block.down(block_ops.swiglu(block.gate_up(block.post_norm(x))))


def replay_hidden(model: LimiteLM, ids: torch.Tensor, *, cache: ReplayContextCache | None = None, checkpoint_layers: bool = True,
                  query_tile: int = 1024, trainable_mode: str = "full") -> torch.Tensor:
    context = cache.prepare(model, ids, trainable_mode) if cache is not None and cache.enabled else _build_context(model, ids, None)
    x = model.embed(ids)
    recompute = checkpoint_layers and torch.is_grad_enabled()
    for i, block in enumerate(model.layers):
        ve = model.value_embeds[str(i)](ids) if str(i) in model.value_embeds else None
        if recompute:
            x = checkpoint(_layer, block, x, ve, context.cos, context.sin, query_tile, use_reentrant=False)
        else:
            x = _layer(block, x, ve, context.cos, context.sin, query_tile)
    return model.norm(x)


def replay_loss(model: LimiteLM, ids, labels, *, cache=None, chunk_size: int = 512, query_tile: int = 1024) -> dict:
    """Mean negative log-likelihood (and entropy) over labelled positions (label -1: ignored) with the vocabulary
    projected chunk by chunk."""
    hidden = replay_hidden(model, ids, cache=cache, query_tile=query_tile)
    out = chunked_logits_processor(model.lm_head, hidden, logprob_entropy_processor, {"labels": labels.clamp_min(0)}, chunk_size=chunk_size)
    valid = labels.ne(-1)
    count = valid.sum().clamp_min(1)
    return {"loss": -(out["log_probs"] * valid).sum() / count, "entropy": (out["entropy"] * valid).sum() / count, "tokens": int(valid.sum())}


def retained_activation_bytes(config, batch: int, length: int, *, bytes_per_element: int = 2, checkpoint_layers: bool = True) -> int:
    """What stays alive between forward and backward: with layer checkpoints, one [B, T, hidden] input per layer plus the
    value-embedding lookups; without, roughly every projection output of every layer."""
    c = config
    tokens = batch * length
    if checkpoint_layers:
        per_layer = c.hidden_size
        extra = len(c.ve_layers) * c.num_key_value_heads * c.head_dim
        return (per_layer * c.num_hidden_layers + extra + c.hidden_size) * tokens * bytes_per_element
    qkv = (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim
    per_layer = 4 * c.hidden_size + qkv + c.num_attention_heads * c.head_dim + 3 * c.intermediate_size
    return per_layer * c.num_hidden_layers * tokens * bytes_per_element
