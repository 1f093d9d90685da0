"""Closed-form parameter counts and a pipeline split for the Qwen3.8 family (27B dense, quarter, Flash-Next).

``parameter_count_contract(config)`` gives the number of parameters of every component from the geometry alone, so a
launcher can check a configuration (and a built model against it) before anything is allocated; ``pipeline_split`` cuts
the decoder into contiguous stages whose parameter loads are as even as possible, with the embedding (and the hashed
per-layer-embedding tables) on the first stage and the final norm, head and multi-token-prediction block on the last.
The reference carries such a contract for its Flash-Next model (src/archlab/architectures/qwen38_flash_next_full.py:
872-940) and splits it by a fixed layer table; here both follow from the configuration.
"""
from __future__ import annotations

from .qwen38 import Qwen38Config, Qwen38LM


def _gdn(c: Qwen38Config) -> int:
    qw, vw, h = c.linear_qk_heads * c.linear_key_dim, c.linear_v_heads * c.linear_value_dim, c.hidden_size
    fused = 2 * qw + vw
    return (h * fused + h * vw + h * 2 * c.linear_v_heads          # qkv, z, beta / decay logits
            + fused * c.linear_conv_kernel + 2 * c.linear_v_heads   # depthwise conv, a_log, dt_bias
            + c.linear_value_dim + vw * h)                          # per-head output norm, output projection


def _attention(c: Qwen38Config) -> int:
    h, q, kv = c.hidden_size, c.attention_heads * c.attention_head_dim, c.attention_kv_heads * c.attention_head_dim
    n = h * 2 * q + 2 * h * kv + 2 * c.attention_head_dim + q * h   # q + gate, k, v, q / k norms, output projection
    if c.sparse_top_k > 0:
        n += h * c.indexer_heads * c.indexer_dim + h * c.indexer_dim + h * c.indexer_heads
    return n


def _mlp(c: Qwen38Config) -> int:
    h = c.hidden_size
    if c.n_experts == 0:
        return 3 * h * c.intermediate_size
    routed = c.n_experts * (2 * c.moe_intermediate_size * h + h * c.moe_intermediate_size)
    shared = 2 * c.moe_intermediate_size * h + c.moe_intermediate_size * h + (h if c.shared_expert_gated else 0)
    return c.n_experts * h + routed + shared                        # router, routed experts, shared expert (+ its gate)


def layer_parameters(c: Qwen38Config, layer: int, *, force_full: bool = False) -> int:
    full = force_full or (layer + 1) % c.full_attention_interval == 0
    return 2 * c.hidden_size + (_attention(c) if full else _gdn(c)) + _mlp(c)


def parameter_count_contract(c: Qwen38Config, *, ple_owners: int = 1) -> dict[str, int]:
    h = c.hidden_size
    layers = [layer_parameters(c, i) for i in range(c.num_hidden_layers)]
    out = {"embedding": c.vocab_size * h, "layers": sum(layers), "final_norm": h, "lm_head": h * c.vocab_size}
    out["mtp"] = 0
    if c.mtp_layers:
        out["mtp"] = layer_parameters(c, c.num_hidden_layers, force_full=True) + h + ((2 * h + 2 * h * h) if c.mtp_fusion else 0)
    out["ple"] = 0
    if c.ngram_size > 1:
        heads = (c.ngram_size - 1) * c.ngram_heads_per_order
        rows = -(-heads * c.ngram_head_vocab // max(ple_owners, 1))
        out["ple"] = max(ple_owners, 1) * rows * c.ngram_dim + heads * c.ngram_dim * h        # all owners' tables + projection
    out["total"] = sum(out.values())
    out["per_layer"] = layers
    return out


def assert_parameter_contract(model: Qwen38LM) -> dict[str, int]:
    """The built model has exactly the parameters its configuration promises (a single-owner table layout)."""
    want = parameter_count_contract(model.config)
    got = sum(p.numel() for p in model.parameters())
    if got != want["total"]:
        raise ValueError(f"model holds {got} parameters, its configuration promises {want['total']}")
    for i, block in enumerate(model.layers):
        n = sum(p.numel() for p in block.parameters())
        if n != want["per_layer"][i]:
            raise ValueError(f"layer {i} holds {n} parameters, the contract says {want['per_layer'][i]}")
    return want


def pipeline_split(c: Qwen38Config, stages: int) -> list[dict]:
    """Contiguous layer ranges ``[first, last)`` per stage minimising the largest stage load (dynamic programme over the
    layers; loads include the embedding side on stage 0 and the head side on the last stage)."""
    n = c.num_hidden_layers
    if not 1 <= stages <= n:
        raise ValueError("need between 1 and num_hidden_layers stages")
    contract = parameter_count_contract(c)
    per = contract["per_layer"]
    head_side = contract["final_norm"] + contract["lm_head"] + contract["mtp"]
    tail_side = contract["embedding"] + contract["ple"]
    prefix = [0]
    for x in per:
        prefix.append(prefix[-1] + x)
    load = lambda a, b, s: prefix[b] - prefix[a] + (tail_side if s == 0 else 0) + (head_side if s == stages - 1 else 0)
    INF = float("inf")
    best = [[INF] * (n + 1) for _ in range(stages + 1)]
    cut = [[0] * (n + 1) for _ in range(stages + 1)]
    best[0][0] = 0
    for s in range(1, stages + 1):
        for b in range(s, n - (stages - s) + 1):
            for a in range(s - 1, b):
                if best[s - 1][a] == INF:
                    continue
                worst = max(best[s - 1][a], load(a, b, s - 1))
                if worst < best[s][b]:
                    best[s][b], cut[s][b] = worst, a
    bounds, b = [], n
    for s in range(stages, 0, -1):
        bounds.append((cut[s][b], b))
        b = cut[s][b]
    bounds.reverse()
    return [{"stage": s, "first_layer": a, "last_layer": b, "parameters": load(a, b, s),
             "holds": (["embedding"] if s == 0 else []) + (["final_norm", "lm_head", "mtp"] if s == stages - 1 else [])}
            for s, (a, b) in enumerate(bounds)]
