"""What a run records about its numeric precision, and the rules a low-precision run has to meet.

The recorded payload and the rules follow the reference's Qwen3.8 trainers (src/archlab/megatron/qwen38_train.py:38-39,
198-229): ``--precision bf16`` or ``fp4``; an FP4 run pads grouped-expert segments to 64 tokens and MTP token counts to
8, caps a grouped product at 64 experts, needs both sides of a dense weight to be multiples of 128 and keeps routing
logits, scalar gates, normalisation and the loss in BF16.  ``fp8`` is the block-scaled recipe of the V4.1 family.
"""
from __future__ import annotations

PRECISIONS = ("bf16", "fp8", "fp4")
# mesh trainer flag -> contract name
FLAG_TO_PRECISION = {"bf16": "bf16", "fp8_block": "fp8", "fp8_tensor": "fp8", "nvfp4": "fp4"}

_CONTRACTS = {
    "bf16": {
        "compute": "BF16", "recipe": "bf16 operands on the tcgen05 kind::f16 kernels, fp32 accumulation",
        "runtime_backend": "native_bf16", "model_parameters": "BF16 shadows of FP32 masters",
        "optimizer_master_parameters": "FP32, sharded over the data group", "moe_grouped_token_padding_multiple": 256,
        "moe_grouped_linear_max_experts": None, "mtp_token_padding_multiple": 1,
    },
    "fp8": {
        "compute": "FP8 block scaling (e4m3, power-of-two scales: 1 x 128 activations, 128 x 128 weights)",
        "recipe": "forward products on tcgen05 kind::mxf8f6f4 with scale factors in TMEM; straight-through bf16 gradients",
        "runtime_backend": "native_fp8_block", "dense_linear_alignment": 128, "moe_grouped_token_padding_multiple": 256,
        "bf16_exceptions": ["routing logits", "hyper-connection coefficients", "reduction width not divisible by 128",
                            "normalization and loss"],
        "optimizer_master_parameters": "FP32",
    },
    "fp4": {
        "compute": "NVFP4 block scaling (e2m1, e4m3 scale per 16, fp32 tensor scale)",
        "recipe": "forward, data-gradient and weight-gradient products on tcgen05 kind::mxf4nvf4",
        "runtime_backend": "native_nvfp4", "stochastic_rounding": True, "two_dimensional_quantization": True,
        "random_hadamard_transform": "weight-gradient operands, 16 x 16, sign-randomised",
        "moe_grouped_token_padding_multiple": 256, "moe_grouped_linear_max_experts": 64, "mtp_token_padding_multiple": 8,
        "dense_linear_alignment": 128,
        "bf16_exceptions": ["routing logits", "shared-expert scalar gate", "dense linear weights with K or N not divisible by 128",
                            "normalization and loss"],
        "optimizer_master_parameters": "FP32",
    },
}


def precision_contract(precision: str) -> dict:
    if precision not in PRECISIONS:
        raise ValueError(f"precision must be one of {PRECISIONS}")
    return dict(_CONTRACTS[precision], precision=precision)


def check_fp4_geometry(*, hidden_size: int, intermediate_sizes: list[int], num_experts: int = 0, tokens_per_microbatch: int = 0,
                       mtp_tokens: int = 0) -> list[str]:
    """Violations of the FP4 rules for a model geometry (empty list = admissible).  A violated dense-alignment rule is
    not fatal by itself - the layer falls back to BF16 - so it is reported as a note, prefixed ``bf16:``."""
    problems = []
    for width in [hidden_size, *intermediate_sizes]:
        if width % 128:
            problems.append(f"bf16: width {width} is not a multiple of 128; its linears stay in BF16")
    if num_experts > 64:
        problems.append(f"grouped product over {num_experts} experts exceeds the cap of 64; split it into chunks of at most 64")
    if tokens_per_microbatch % 64:
        problems.append(f"{tokens_per_microbatch} tokens per micro-batch is not a multiple of 64")
    if mtp_tokens % 8:
        problems.append(f"{mtp_tokens} MTP tokens is not a multiple of 8")
    return problems


def resume_compatible(recorded: dict, current: dict) -> list[str]:
    """Keys of the precision contract that differ between the run on disk and the resuming process; a resume under
    another precision recipe is refused by the caller."""
    return sorted(k for k in set(recorded) | set(current) if recorded.get(k) != current.get(k))
