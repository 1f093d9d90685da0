"""``arch_family`` -> (config class, model class), construction from checkpoint metadata with
back-compat patching of configurations written before newer fields existed
(src/archlab/model_factory.py:25-435)."""
from __future__ import annotations

import dataclasses
from typing import Any

import torch


def _registry() -> dict[str, tuple[type, type]]:
    from . import deepseek_v41, frontier, kimi, limite, nanochat, qwen35, qwen38, sota

    return {
        "nanochat": (nanochat.GPTConfig, nanochat.GPT),
        "engram": (nanochat.GPTConfig, nanochat.GPT),
        "mhc": (nanochat.GPTConfig, nanochat.GPT),
        "kimi_kda": (kimi.KimiConfig, kimi.KimiLM),
        "kimi_attnres": (kimi.KimiConfig, kimi.KimiLM),
        "qwen35": (qwen35.Qwen35Config, qwen35.Qwen35LM),
        "qwen38_27b_text": (qwen38.Qwen38Config, qwen38.Qwen38LM),
        "qwen38_27b_quarter_text": (qwen38.Qwen38Config, qwen38.Qwen38LM),
        "qwen38_flash_next_quarter": (qwen38.Qwen38Config, qwen38.Qwen38LM),
        "qwen38_tiny": (qwen38.Qwen38Config, qwen38.Qwen38LM),
        "deepseek_v41": (deepseek_v41.V41Config, deepseek_v41.V41LM),
        "frontier": (frontier.FrontierConfig, frontier.FrontierLM),
        "sota": (sota.SotaConfig, sota.SotaLM),
        "fog": (sota.SotaConfig, sota.SotaLM),
        "limite": (limite.LimiteConfig, limite.LimiteLM),
    }


_EAGER_FAMILIES = frozenset({"frontier", "sota", "fog", "limite"})


def families() -> list[str]:
    return sorted(_registry())


def classes_for(arch_family: str) -> tuple[type, type]:
    reg = _registry()
    if arch_family not in reg:
        raise ValueError(f"unknown arch_family {arch_family!r}; known: {', '.join(sorted(reg))}")
    return reg[arch_family]


_DTYPES = {"torch.bfloat16": torch.bfloat16, "torch.float32": torch.float32, "torch.float16": torch.float16}


def patch_config(arch_family: str, kwargs: dict[str, Any]) -> dict[str, Any]:
    """Drop keys the current config class no longer knows (recording them), restore dtypes stored as
    strings, and leave missing keys to the dataclass defaults."""
    cfg_cls, _ = classes_for(arch_family)
    known = {f.name for f in dataclasses.fields(cfg_cls)}
    out, dropped = {}, []
    for k, v in kwargs.items():
        if k not in known:
            dropped.append(k)
            continue
        out[k] = _DTYPES.get(v, v) if isinstance(v, str) else v
    if "arch_family" in known:
        out.setdefault("arch_family", arch_family)
    out_dropped = sorted(dropped)
    return out if not out_dropped else {**out, "__dropped__": out_dropped}


def build_model(arch_family: str, config: dict[str, Any] | None = None, *, device="cpu", init: bool = True, **model_kwargs):
    cfg_cls, model_cls = classes_for(arch_family)
    kw = patch_config(arch_family, dict(config or {}))
    kw.pop("__dropped__", None)
    cfg = cfg_cls(**kw)
    if arch_family in _EAGER_FAMILIES:
        # constructors of these families set scalar gains, biases and fixed feature banks themselves
        model = model_cls(cfg, **model_kwargs).to(device)
    else:
        with torch.device("meta"):
            model = model_cls(cfg, **model_kwargs)
        model.to_empty(device=device)
    if init and hasattr(model, "init_weights"):
        model.init_weights()
    return model


def build_from_meta(meta: dict[str, Any], *, device="cpu"):
    """``meta`` as written beside a checkpoint: ``{"model_config": {...}}`` with an optional ``arch_family``."""
    cfg = dict(meta["model_config"])
    family = cfg.get("arch_family", meta.get("arch_family", "nanochat"))
    return build_model(family, cfg, device=device, init=False)
