"""``arch_family`` -> (config class, model class), construction from checkpoint metadata with
back-compat patching of configurations written before newer fields existed
(src/archlab/model_factory.py:25-435)."""
from __future__ import annotations

import dataclasses
from typing import Any

import torch


def _registry() -> dict[str, tuple[type, type]]:
    from . import deepseek_v41, frontier, kimi, limite, nanochat, nanochat_variants, qwen35, qwen38, sota

    return {
        "nanochat": (nanochat.GPTConfig, nanochat.GPT),
        "engram": (nanochat_variants.EngramGPTConfig, nanochat_variants.EngramGPT),
        "mhc": (nanochat_variants.MhcGPTConfig, nanochat_variants.MhcGPT),
        "deepseek_dsa": (nanochat_variants.DsaGPTConfig, nanochat_variants.DsaGPT),
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


_EAGER_FAMILIES = frozenset({"frontier", "sota", "fog", "limite", "engram"})   # engram: hash tables are built from data


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
        if hasattr(model, "_tag"):           # materialisation made new Parameter objects: optimizer tags go on again
            model._tag()
    if init and hasattr(model, "init_weights"):
        model.init_weights()
    return model


def build_from_meta(meta: dict[str, Any], *, device="cpu"):
    """``meta`` as written beside a checkpoint: ``{"model_config": {...}}`` with an optional ``arch_family``."""
    cfg = dict(meta["model_config"])
    family = cfg.get("arch_family", meta.get("arch_family", "nanochat"))
    return build_model(family, cfg, device=device, init=False)


# ------------------------------------------------------------------------------------------------
# campaign arms -> this package's families
# ------------------------------------------------------------------------------------------------
_ARM_FAMILY = {"engram": "engram", "mhc": "mhc", "deepseek_dsa": "deepseek_dsa", "sota_pool": "sota", "pareto_combo": "sota", "combo_search": "sota", "frontier_pool": "frontier",
               "kimi_kda": "kimi_kda", "kimi_attnres": "kimi_attnres", "nanochat": "nanochat"}
_FRONTIER_NAMES = {"glm_mla_muon_split": "glm_mla"}


def campaign_arm_config(kwargs: dict[str, Any]) -> tuple[str, dict[str, Any]]:
    """Translates the model arguments of a frozen campaign arm (``contracts.campaigns.*_model_config_kwargs``:
    depth / aspect ratio / head width plus one mechanism, src/archlab/model_factory.py:243-350) into a family of
    this package and the fields of its config class.  Arms whose mechanism has no model here (Engram memory,
    multi-stream hyper-connections and the small DSA model as nanochat-sized families, gated attention) are
    refused by name rather than silently built as the baseline."""
    kw = dict(kwargs)
    arm = kw.pop("arch_family", "nanochat")
    if arm not in _ARM_FAMILY:
        raise NotImplementedError(f"campaign family {arm!r} has no nanochat-sized model in this package")
    depth, head_dim = int(kw.pop("depth")), int(kw.pop("head_dim"))
    width = -(-depth * int(kw.pop("aspect_ratio")) // head_dim) * head_dim
    cfg: dict[str, Any] = {"n_layer": depth, "n_embd": width, "n_head": width // head_dim,
                           "sequence_len": int(kw.pop("max_seq_len", 2048)), "vocab_size": int(kw.pop("vocab_size", 32768))}
    family = _ARM_FAMILY[arm]
    if family == "sota":
        variant = kw.pop("sota_variant", None) or kw.pop("search_mlp", None) or "baseline"
        variant = {"bank_of_values": "bov", "differential_attention": "diff_attn", "dynamic_tanh": "dyt"}.get(variant, variant)
        if variant not in ("baseline", "xielu", "colu", "dyt", "canon", "bov", "diff_attn", "gated_relu", "qat",
                           "gated_attention", "exclusive_attention"):
            raise NotImplementedError(f"mechanism {variant!r} is not part of the SoTA pool of this package")
        cfg["mechanisms"] = () if variant == "baseline" else (variant,)
        if "colu_dim" in kw:
            cfg["colu_dim"] = kw.pop("colu_dim")
        if "bov_target_fraction" in kw:
            cfg["bov_fraction"] = kw.pop("bov_target_fraction")
        if kw.get("fog_variant") and arm == "fog":
            cfg["fog_variant"] = kw["fog_variant"]
    elif family == "frontier":
        v = kw.pop("frontier_variant", "baseline")
        cfg["variant"] = _FRONTIER_NAMES.get(v, v)
        cfg["relative_dim"] = kw.pop("relative_dim", 16)
    elif family == "kimi_kda":
        cfg.update(kda_pattern=kw.pop("kda_pattern", "KKKG"), kda_variant=kw.pop("kda_variant", "kimi_linear"),
                   kda_force_final_global=kw.pop("kda_force_final_global", True))
    elif family == "kimi_attnres":
        cfg.update(attnres_block=kw.pop("attn_res_block_size", 2), attnres_heads=kw.pop("attn_res_heads", 1))
    elif family in ("nanochat", "engram", "mhc", "deepseek_dsa"):
        cfg.update(n_kv_head=cfg["n_head"], window_pattern=kw.pop("window_pattern", "L"))
        prefix = {"engram": "engram_", "mhc": "mhc_", "deepseek_dsa": "dsa_"}.get(family, "\0")
        cfg.update({k: kw.pop(k) for k in list(kw) if k.startswith(prefix)})
    return family, cfg


def build_campaign_arm(kwargs: dict[str, Any], *, device="cpu"):
    family, cfg = campaign_arm_config(kwargs)
    return build_model(family, cfg, device=device)
