"""Request-local incremental form of a stream adapter: bounded key/value state, contiguous prefill chunks or single
tokens, the same parameters and the same residual equation as the training-time module.

The serving engine owns one instance per request and adapter site and hands it the post-attention stream state
``[B, L, streams * C]`` of every new chunk together with the chunk's start position.  The instance projects only the new
tokens (RoPE at their absolute positions), appends their keys and values to windows of at most ``long_window`` (and
``short_window``) cached positions, and runs the windowed core on [cache | chunk] in one call, so a prefill chunk is one
kernel launch rather than one per token.  Positions must be contiguous; a failed call leaves position and cache as
they were; there is no prefix sharing, padding or rollback, and training mode is refused.
(The reference's per-token FP32 oracle of the same contract: src/archlab/architectures/deepseek_v41_incremental.py:19-129.)
"""
from __future__ import annotations

import torch

from ..models.adapters import StreamAdapter
from ..models.blocks import GatedStreamResidual


class IncrementalStreamAdapter:
    def __init__(self, adapter: StreamAdapter):
        if not isinstance(adapter, StreamAdapter) or adapter.c.mechanism not in ("simplicial", "normal"):
            raise TypeError("expected a simplicial or normal stream adapter")
        self.adapter = adapter
        self.reset()

    def reset(self) -> None:
        self.position = 0
        self._cache: dict[str, torch.Tensor] = {}
        self._signature = None

    @property
    def cache_lengths(self) -> dict[str, int]:
        return {name: t.shape[1] for name, t in self._cache.items()}

    def _windows(self) -> dict[str, int]:
        c = self.adapter.c
        if c.mechanism == "normal":
            return {"k0": c.long_window, "v0": c.long_window}
        return {"k0": c.short_window, "v0": c.short_window, "k1": c.long_window, "v1": c.long_window}

    @torch.inference_mode()
    def __call__(self, packed: torch.Tensor, *, start_position: int) -> torch.Tensor:
        a, c = self.adapter, self.adapter.c
        if a.training:
            raise ValueError("the incremental adapter needs eval mode")
        if type(start_position) is not int or start_position != self.position:
            raise ValueError("non-contiguous position; reset the cache for a new request")
        if packed.ndim != 3 or min(packed.shape) < 1 or packed.shape[-1] != c.streams * c.hidden_size:
            raise ValueError("expected unpadded [batch, sequence, streams * width]")
        signature = (packed.shape[0], packed.device, packed.dtype)
        if self._signature is not None and signature != self._signature:
            raise ValueError("batch / device / dtype changed within a request")
        x, packed, weights = a.read(packed)
        x = x.to(packed.dtype)
        q, ks, vs = a.project(x, offset=self.position)
        L = packed.shape[1]
        fresh = {f"k{i}": k for i, k in enumerate(ks)} | {f"v{i}": v for i, v in enumerate(vs)}
        # every name attends over [cached | new]; the short streams need only their own window in front of the chunk, but
        # the core takes equally long key sequences, so short ones are left-padded with zeros that their window never reaches
        joined = {n: torch.cat((self._cache[n], t), dim=1) if n in self._cache else t for n, t in fresh.items()}
        S = max(t.shape[1] for t in joined.values())
        padded = {n: t if t.shape[1] == S else torch.cat((t.new_zeros(t.shape[0], S - t.shape[1], *t.shape[2:]), t), dim=1) for n, t in joined.items()}
        y = a.attend(q, [padded[f"k{i}"] for i in range(len(ks))], [padded[f"v{i}"] for i in range(len(vs))])
        out = GatedStreamResidual.inject(packed, a.finish(x, y), weights.to(packed.dtype))
        # commit only after everything succeeded; cloned slices, so a long prefill does not keep its storage alive
        self._cache = {n: t[:, -(w - 1):].clone() if w > 1 else t[:, :0].clone() for n, t in joined.items() for w in (self._windows()[n],)}
        self._signature = signature
        self.position += L
        return out
