"""Runtime backends of the Qwen3.8 family: which GEMM path every projection takes, decided once, reported, and bound
by shape rules that can be checked before a run.

``runtime_backend``:

* ``native``        plain PyTorch linears (the CPU-testable form);
* ``kernels_bf16``  every eligible linear on the tcgen05 bf16 GEMM (``ops.native_linear``);
* ``fp8_block``     128-block-scaled FP8 products for eligible linears, bf16 kernels for the exceptions;
* ``nvfp4``         NVFP4 products (Hadamard + stochastic rounding on the gradient side) for eligible linears.

Shape rules of the block-scaled backends: both weight sides must be multiples of 128 (else the layer is a *bf16
exception*, listed with its reason); routing logits, scalar gates and the output head stay in bf16 by role; grouped
expert GEMMs run over 128-row tiles, so every expert's row segment is padded up to a multiple of 128 and
``expert_padding`` says what that costs for a given routing load.  (The reference selects ``te_bf16`` / ``te_fp4`` through
a library and states its own rules -- dims % 128, expert splits padded to 64, at most 64 experts per grouped call:
src/archlab/architectures/qwen38_flash_next.py:152-228,284-301.)
"""
from __future__ import annotations

import torch

from .qwen38 import Qwen38Config, Qwen38LM

RUNTIME_BACKENDS = ("native", "kernels_bf16", "fp8_block", "nvfp4")
ALIGNMENT, GROUP_TILE_ROWS = 128, 128


def projection_shapes(c: Qwen38Config) -> dict[str, tuple[int, int]]:
    """(out, in) of every distinct projection of the configuration, by role."""
    qw, vw = c.linear_qk_heads * c.linear_key_dim, c.linear_v_heads * c.linear_value_dim
    aq, akv = c.attention_heads * c.attention_head_dim, c.attention_kv_heads * c.attention_head_dim
    shapes = {"gdn.qkv": (2 * qw + vw, c.hidden_size), "gdn.z": (vw, c.hidden_size), "gdn.out": (c.hidden_size, vw),
              "attention.q_gate": (2 * aq, c.hidden_size), "attention.k": (akv, c.hidden_size), "attention.v": (akv, c.hidden_size),
              "attention.out": (c.hidden_size, aq)}
    if c.n_experts:
        shapes |= {"experts.gate_up": (2 * c.moe_intermediate_size, c.hidden_size), "experts.down": (c.hidden_size, c.moe_intermediate_size)}
    else:
        shapes |= {"mlp.gate": (c.intermediate_size, c.hidden_size), "mlp.up": (c.intermediate_size, c.hidden_size),
                   "mlp.down": (c.hidden_size, c.intermediate_size)}
    return shapes


def shape_rules(c: Qwen38Config, backend: str) -> dict:
    """Which roles the backend covers at this geometry; nothing is built."""
    if backend not in RUNTIME_BACKENDS:
        raise ValueError(f"runtime_backend must be one of {RUNTIME_BACKENDS}")
    shapes = projection_shapes(c)
    if backend in ("native", "kernels_bf16"):
        return {"backend": backend, "covered": sorted(shapes), "bf16_exceptions": {}}
    bad = {role: f"{o} x {i} is not {ALIGNMENT}-aligned" for role, (o, i) in shapes.items() if o % ALIGNMENT or i % ALIGNMENT}
    return {"backend": backend, "covered": sorted(set(shapes) - set(bad)), "bf16_exceptions": bad}


def expert_padding(rows_per_expert, tile: int = GROUP_TILE_ROWS) -> dict:
    """Rows the grouped GEMM really runs for a routing load: every non-empty expert segment rounds up to whole tiles."""
    rows = [int(r) for r in rows_per_expert]
    padded = [-(-r // tile) * tile for r in rows]
    total = sum(rows)
    return {"rows": total, "padded_rows": sum(padded), "tiles": sum(p // tile for p in padded),
            "overhead": (sum(padded) - total) / total if total else 0.0}


def apply_runtime_backend(model: Qwen38LM, backend: str) -> dict:
    """Binds the model's linears to ``backend`` in place (once) and returns the report that a run records."""
    if backend not in RUNTIME_BACKENDS:
        raise ValueError(f"runtime_backend must be one of {RUNTIME_BACKENDS}")
    if getattr(model, "_runtime_backend", None) is not None:
        raise ValueError(f"the model already runs on {model._runtime_backend!r}")
    report = {"backend": backend, "converted": [], "bf16_exceptions": {}}
    if backend == "kernels_bf16":
        from ..ops.native_linear import convert_linears

        report["converted"] = convert_linears(model)
    elif backend in ("fp8_block", "nvfp4"):
        from ..ops.blockscaled import convert_linears

        # by role only the head, the router and the scalar shared-expert gate stay in bf16; ``mlp.gate`` and ``q_gate`` are
        # full projections despite their names
        done = convert_linears(model, backend, skip=("lm_head", "router", "shared_gate"))
        report.update(converted=done["converted"], bf16_exceptions=done["bf16_exceptions"])
    report["expected"] = shape_rules(model.config, backend)
    model._runtime_backend = backend
    return report
