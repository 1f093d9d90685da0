"""2-simplicial attention as a drop-in token mixer for the speedrun GPT block.

The reference only *inserts* simplicial branches into Qwen / V4.1 / Megatron models
(src/archlab/architectures/qwen35_insertion.py:70-176, megatron/simplicial_attention.py:36-122);
the benchmark configs additionally swap one GPT layer's attention for it, so this module gives the
layer the same q / k / v / proj naming as ``CausalSelfAttention`` plus a second key / value branch
(``c_k2`` / ``c_v2``).  q, k1 and k2 get RoPE + parameter-free RMSNorm (gain 1.2 on q and k1 only,
so the trilinear score has the same scale budget as a bilinear one); values are left untouched.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops.simplicial import simplicial_attention


class SimplicialSelfAttention(nn.Module):
    def __init__(self, config, layer_idx: int):
        super().__init__()
        from .nanochat import CastLinear

        self.config, self.layer_idx = config, layer_idx
        C, H, Hkv, D = config.n_embd, config.n_head, config.n_kv_head, config.head_dim
        self.c_q = CastLinear(C, H * D)
        self.c_k = CastLinear(C, Hkv * D)
        self.c_v = CastLinear(C, Hkv * D)
        self.c_k2 = CastLinear(C, Hkv * D)
        self.c_v2 = CastLinear(C, Hkv * D)
        self.c_proj = CastLinear(C, C)
        self.ve_gate = None
        self.w1, self.w2 = config.simplicial_w1, config.simplicial_w2

    def forward(self, x, ve, cos, sin, window):
        from .nanochat import apply_rope, rms_norm

        B, T, _ = x.shape
        cfg = self.config
        H, Hkv, D = cfg.n_head, cfg.n_kv_head, cfg.head_dim
        q = self.c_q(x).view(B, T, H, D)
        k1 = self.c_k(x).view(B, T, Hkv, D)
        v1 = self.c_v(x).view(B, T, Hkv, D)
        k2 = self.c_k2(x).view(B, T, Hkv, D)
        v2 = self.c_v2(x).view(B, T, Hkv, D)
        q = rms_norm(apply_rope(q, cos, sin)) * 1.2
        k1 = rms_norm(apply_rope(k1, cos, sin)) * 1.2
        k2 = rms_norm(apply_rope(k2, cos, sin))
        y = simplicial_attention(q, k1, k2, v1, v2, self.w1, self.w2)
        return self.c_proj(y.contiguous().view(B, T, -1))
