"""Single-GPU inference of a model whose experts and hashed tables do not fit the GPU: they stay ENCODED in (pinned)
host memory and only what a batch touches is decoded on the device.

* ``DecodedExpertCache``: an LRU of decoded expert weight sets bounded in BYTES.  A miss copies the expert's encoded
  matrices and scales to the device (non-blocking from pinned memory), decodes them there and evicts least-recently-used
  experts until the new one fits; an expert larger than the whole budget is served but not kept.  Hits, misses and
  evictions are counted, since the hit rate decides whether offloaded inference is usable at all.
* ``OffloadedExperts``: runs the routed experts of one MoE layer with weights from the cache; the arithmetic (clamped
  SwiGLU, routing-probability scaling, fp32 accumulation in ascending expert order) is the training-time arithmetic.
* ``encoded_row_lookup``: gathers ENCODED rows (fp8 payload + per-block scales) of a host table by index on the CPU,
  ships only those rows and decodes them on the device; indices outside the table are an error, not a wrap-around.
(Reference: src/archlab/automodel/deepseek_v41_local_inference.py:37-100.)
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Callable

import torch
import torch.nn.functional as F


def _nbytes(tensors: dict[str, torch.Tensor]) -> int:
    return sum(t.numel() * t.element_size() for t in tensors.values())


class DecodedExpertCache:
    def __init__(self, max_bytes: int, decode: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], device="cpu"):
        self.max_bytes, self.decode, self.device = int(max_bytes), decode, torch.device(device)
        self.entries: OrderedDict = OrderedDict()
        self.bytes = self.hits = self.misses = self.evictions = 0

    def get(self, key, encoded: dict[str, tuple[torch.Tensor, torch.Tensor]]) -> dict[str, torch.Tensor]:
        """``encoded``: name -> (payload, scales) on the host."""
        if key in self.entries:
            self.hits += 1
            self.entries.move_to_end(key)
            return self.entries[key]
        self.misses += 1
        decoded = {name: self.decode(w.to(self.device, non_blocking=True), s.to(self.device, non_blocking=True)) for name, (w, s) in encoded.items()}
        size = _nbytes(decoded)
        while self.entries and self.bytes + size > self.max_bytes:
            _, gone = self.entries.popitem(last=False)
            self.bytes -= _nbytes(gone)
            self.evictions += 1
        if size <= self.max_bytes:
            self.entries[key] = decoded
            self.bytes += size
        return decoded

    def stats(self) -> dict:
        total = self.hits + self.misses
        return {"hits": self.hits, "misses": self.misses, "evictions": self.evictions, "resident_experts": len(self.entries), "resident_bytes": self.bytes,
                "hit_rate": self.hits / total if total else 0.0}


class OffloadedExperts:
    """``encoded[e] = {"gate_up": (payload, scales), "down": (payload, scales)}`` for the experts of one layer."""

    def __init__(self, layer_key, encoded: list[dict], cache: DecodedExpertCache, *, swiglu_limit: float | None = None):
        self.layer_key, self.encoded, self.cache, self.limit = layer_key, encoded, cache, swiglu_limit

    @torch.no_grad()
    def __call__(self, x: torch.Tensor, indices: torch.Tensor, probabilities: torch.Tensor) -> torch.Tensor:
        """x [T, D]; indices / probabilities [T, k] -> fp32 [T, D]."""
        out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
        for e in torch.unique(indices).tolist():                      # ascending expert id: a fixed summation order
            rows, slots = torch.where(indices == e)
            w = self.cache.get((self.layer_key, e), self.encoded[e])
            gate, up = F.linear(x[rows], w["gate_up"].to(x.dtype)).float().chunk(2, -1)
            if self.limit is not None:
                gate, up = gate.clamp(max=self.limit), up.clamp(-self.limit, self.limit)
            hidden = F.silu(gate) * up * probabilities[rows, slots, None].float()
            out.index_add_(0, rows, F.linear(hidden.to(x.dtype), w["down"].to(x.dtype)).float())
        return out


def encoded_row_lookup(payload: torch.Tensor, scales: torch.Tensor, indices: torch.Tensor, *, block: int, dim: int, out_dtype=torch.bfloat16) -> torch.Tensor:
    """``payload`` [rows, dim] (fp8 or any 1-byte float format) and ``scales`` [rows, dim / block] live on the host."""
    ids = indices.reshape(-1).cpu()
    if bool(((ids < 0) | (ids >= payload.shape[0])).any()):
        raise ValueError("table index outside the original table")
    dev = indices.device
    values = payload.view(torch.uint8).index_select(0, ids).to(dev, non_blocking=True).view(payload.dtype)       # integer views: CPU gathers lack fp8 kernels
    scale = scales.view(torch.uint8).index_select(0, ids).to(dev, non_blocking=True).view(scales.dtype) if scales.element_size() == 1 else scales.index_select(0, ids).to(dev)
    decoded = values.float().unflatten(-1, (-1, block)) * scale.float().unsqueeze(-1)
    return decoded.flatten(-2).to(out_dtype).reshape(*indices.shape, dim)
