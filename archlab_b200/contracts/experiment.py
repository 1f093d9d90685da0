"""Typed experiment contract, overlay / override merge and fail-closed science validators.

Mirrors the behaviour of the reference's ``archlab.training.config`` (``Experiment`` dataclass
:18-50, ``read_experiment`` :53-106, composition :109-146, ``validate_science`` :149-349,
``fingerprint`` :352-353) without OmegaConf / Hydra: recipes and overlays are plain YAML merged
in order onto the dataclass defaults, trailing ``key=value`` overrides update typed fields, and
``settings.<dotted.path>=value`` writes a literal path of the composed trainer configuration tree
(which is struct-checked: an unknown path is an error, never a silent new key).
``${oc.env:NAME[,default]}`` interpolations are resolved when the tree is composed.
"""
from __future__ import annotations

import copy
import dataclasses
import hashlib
import json
import math
import os
import re
from dataclasses import dataclass, field, fields
from pathlib import Path
from typing import Any

import yaml

from .performance import ThroughputContract

MISSING = "???"
FAMILIES = {"limite", "muse_glimmer", "qwen3_5", "speedrun"}
VARIANTS = {"normal", "simplicial", "linsimp", "triadic"}
INTERVENTIONS = {"insert_attention", "replace_attention", "none"}
ENGINES = {"megatron", "dp"}
ATTENTION = {"native", "tilelang", "te"}
EXECUTION = {"sync", "colocate_async"}
CONFIG_ROOT = Path(__file__).resolve().parent.parent / "config_tree"


@dataclass
class AgenticPilot:
    max_turn_tokens: int = 8192
    step_limit: int = 500
    minimum_prompt_groups: int = 2
    minimum_completed_verifiers: int = 8
    minimum_tool_calls: int = 1
    minimum_observation_tokens: int = 1
    minimum_reward_contrast_groups: int = 1
    maximum_truncated_trajectories: int = 0


@dataclass
class Experiment:
    name: str = MISSING
    family: str = "limite"
    variant: str = "normal"
    intervention: str = "insert_attention"
    engine: str = "megatron"
    attention: str = "tilelang"
    execution: str = "colocate_async"
    native_context: int = 131072
    parent_checkpoint: str = MISSING
    parent_stage: str = "adapter_sft"
    parent_tokens: int | None = 2_000_158_720
    publisher_manifest: str | None = None
    data_manifest: str = MISSING
    resume_checkpoint: str | None = None
    maximum_policy_lag: int = 1
    pilot: AgenticPilot | None = None
    throughput: ThroughputContract = field(default_factory=ThroughputContract)
    settings: dict[str, Any] = field(default_factory=dict)


# ------------------------------------------------------------------------------------------------
# merge
# ------------------------------------------------------------------------------------------------
def parse_scalar(raw: str) -> Any:
    """YAML scalar / flow syntax, the same value grammar a dotlist override uses."""
    try:
        return yaml.safe_load(raw)
    except yaml.YAMLError:
        return raw


def _coerce(value: Any, typ: Any, label: str) -> Any:
    if value is None:
        return None
    origin = getattr(typ, "__origin__", None)
    if typ in (int, "int") or str(typ) in ("int | None", "int"):
        if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value:
            raise ValueError(f"{label} must be an integer")
        return int(value)
    if typ in (str,) or str(typ) in ("str | None", "str"):
        return str(value)
    if origin is dict or typ is dict:
        if not isinstance(value, dict):
            raise ValueError(f"{label} must be a mapping")
        return dict(value)
    return value


def _build_dataclass(cls, data: dict, label: str):
    known = {f.name: f for f in fields(cls)}
    unknown = set(data) - set(known)
    if unknown:
        raise ValueError(f"unknown key(s) in {label}: {', '.join(sorted(unknown))}")
    kwargs = {}
    for name, f in known.items():
        if name not in data:
            continue
        v = data[name]
        if name == "pilot":
            kwargs[name] = None if v is None else _build_dataclass(AgenticPilot, dict(v), "pilot")
        elif name == "throughput":
            kwargs[name] = _build_dataclass(ThroughputContract, dict(v or {}), "throughput")
        else:
            kwargs[name] = _coerce(v, f.type, f"{label}.{name}" if label else name)
    return cls(**kwargs)


def _deep_merge(base: dict, update: dict) -> dict:
    for k, v in update.items():
        if isinstance(v, dict) and isinstance(base.get(k), dict):
            _deep_merge(base[k], v)
        else:
            base[k] = copy.deepcopy(v)
    return base


def _set_dotted(tree: dict, dotted: str, value: Any, *, struct: bool, label: str = "") -> None:
    node = tree
    parts = dotted.split(".")
    for i, part in enumerate(parts[:-1]):
        if not isinstance(node, dict) or part not in node:
            if struct:
                raise KeyError(f"unknown configuration path {label}{'.'.join(parts[:i + 1])}")
            node = node.setdefault(part, {})
        else:
            node = node[part]
    if struct and (not isinstance(node, dict) or parts[-1] not in node):
        raise KeyError(f"unknown configuration path {label}{dotted}")
    node[parts[-1]] = value


def read_experiment(path: str | Path, overrides: list[str] | tuple[str, ...] = (), *,
                    overlays: list[Path] | tuple[Path, ...] = ()) -> Experiment:
    data: dict = {}
    for src in (path, *overlays):
        loaded = yaml.safe_load(Path(src).read_text(encoding="utf-8")) or {}
        if not isinstance(loaded, dict):
            raise ValueError(f"recipe must be a mapping: {src}")
        settings = loaded.pop("settings", None)
        _deep_merge(data, loaded)
        if settings:
            # settings keys are literal dotted upstream paths; later files replace whole values
            data.setdefault("settings", {}).update(settings)
    for ov in overrides:
        key, sep, raw = ov.partition("=")
        if not sep or not key:
            raise ValueError("overrides must use key=value")
        value = parse_scalar(raw)
        if key.startswith("settings."):
            data.setdefault("settings", {})[key[len("settings."):]] = value
        else:
            _set_dotted(data, key, value, struct=False)
    # experiment fields interpolate environment variables like the trainer tree does; a variable that is not set
    # (and has no default) stays as written, so a recipe can be read and checked without its deployment environment
    for key in list(data):
        if key != "settings":
            data[key] = _resolve_env(data[key], os.environ, strict=False)
    exp = _build_dataclass(Experiment, data, "")
    for req in ("name", "parent_checkpoint", "data_manifest"):
        if getattr(exp, req) == MISSING:
            raise ValueError(f"missing mandatory value: {req}")
    validate_experiment(exp)
    return exp


def validate_experiment(e: Experiment) -> None:
    """Cross-field rules of the typed contract (reference :68-105)."""
    e.throughput.validate()
    if e.family not in FAMILIES:
        raise ValueError("unknown model family")
    if e.family == "limite" and e.engine != "megatron":
        raise ValueError("the primary execution engine is megatron")
    if e.engine not in ENGINES:
        raise ValueError("engine must be megatron or dp")
    if e.attention not in ATTENTION:
        raise ValueError("attention must be native, tilelang or te")
    if e.execution not in EXECUTION:
        raise ValueError("execution must be sync or colocate_async")
    if e.variant not in VARIANTS:
        raise ValueError("unknown architecture variant")
    if e.intervention not in INTERVENTIONS:
        raise ValueError("unknown architecture intervention")
    if e.native_context <= 0:
        raise ValueError("native_context must be positive")
    if e.maximum_policy_lag < 0:
        raise ValueError("maximum_policy_lag must be nonnegative")
    if e.family == "speedrun":
        return   # pre-training runs on this framework's own trainer; no RL lineage rules apply
    if e.family != "qwen3_5" and e.maximum_policy_lag != 1:
        raise ValueError("the existing Limite and Muse pilots permit at most one policy version of lag")
    if e.resume_checkpoint and e.family != "qwen3_5":
        raise ValueError("the existing Limite and Muse pilots require fresh RL")
    if e.family in {"muse_glimmer", "qwen3_5"}:
        if (e.engine != "dp" or e.variant != "normal" or e.attention != "native" or e.intervention != "none"
                or e.parent_stage != "published_checkpoint" or e.parent_tokens is not None
                or not e.publisher_manifest):
            raise ValueError("native control requires DP, unchanged publisher weights and an asset manifest")
    elif e.intervention == "none":
        raise ValueError("Limite requires its explicit attention intervention")
    elif e.parent_stage == "package_sft":
        if (e.intervention != "replace_attention" or e.variant != "simplicial" or e.attention != "tilelang"
                or e.parent_tokens is not None):
            raise ValueError("package SFT replacement uses simplicial TileLang and receipt-derived token budgets")
    elif e.parent_stage not in {"adapter_sft", "full_sft"} or e.parent_tokens is None or e.parent_tokens <= 0:
        raise ValueError("this fresh RL pilot requires an explicit SFT token endpoint")
    if e.intervention == "replace_attention" and e.parent_stage != "package_sft":
        raise ValueError("attention replacement RL requires a trained package SFT endpoint")


def experiment_dict(e: Experiment) -> dict:
    return dataclasses.asdict(e)


def fingerprint(config: Any) -> str:
    """sha256 of the canonical JSON of a resolved configuration."""
    return hashlib.sha256(json.dumps(config, sort_keys=True, default=str).encode()).hexdigest()


# ------------------------------------------------------------------------------------------------
# composition of the trainer configuration tree
# ------------------------------------------------------------------------------------------------
class Tree(dict):
    """dict with attribute access (read-only convenience for the validators)."""

    def __getattr__(self, k):
        try:
            v = self[k]
        except KeyError as e:
            raise AttributeError(k) from e
        return Tree(v) if isinstance(v, dict) and not isinstance(v, Tree) else v


_INTERP = re.compile(r"\$\{oc\.env:([A-Za-z_][A-Za-z0-9_]*)(?:,([^}]*))?\}")


def _resolve_env(value: Any, environ, strict: bool = True) -> Any:
    if isinstance(value, dict):
        return {k: _resolve_env(v, environ, strict) for k, v in value.items()}
    if isinstance(value, list):
        return [_resolve_env(v, environ, strict) for v in value]
    if isinstance(value, str):
        whole = _INTERP.fullmatch(value)

        def sub(m):
            got = environ.get(m.group(1), m.group(2))
            if got is None:
                if not strict:
                    return m.group(0)
                raise ValueError(f"environment variable {m.group(1)} is not set and has no default")
            return str(got)

        if whole:
            return parse_scalar(sub(whole))
        return _INTERP.sub(sub, value)
    return value


def _find_missing(tree: Any, prefix: str = "") -> list[str]:
    out = []
    if isinstance(tree, dict):
        for k, v in tree.items():
            out += _find_missing(v, f"{prefix}{k}.")
    elif tree == MISSING:
        out.append(prefix[:-1])
    return out


def compose_trainer(experiment: Experiment, config_root: Path | None = None, *, environ=None,
                    validate: bool = True) -> dict:
    """Build the resolved trainer configuration: base tree for the engine, then every
    ``settings`` entry written to its literal dotted path (struct-checked), then the experiment-
    derived fields, environment interpolation and the science validators."""
    root = Path(config_root) if config_root is not None else CONFIG_ROOT
    name = "ppo_trainer.yaml" if experiment.engine == "dp" else "train.yaml"
    tree = yaml.safe_load((root / name).read_text(encoding="utf-8"))
    tree["model_engine"] = experiment.engine
    for key, value in experiment.settings.items():
        try:
            _set_dotted(tree, key, copy.deepcopy(value), struct=True, label="settings.")
        except KeyError as e:
            raise ValueError(str(e.args[0])) from e
    tree["trainer"]["experiment_name"] = experiment.name
    tree["trainer"]["use_v1"] = True
    tree["trainer"]["v1"]["trainer_mode"] = experiment.execution
    if not tree["reward"]["reward_model"]["enable"]:
        tree["reward"]["reward_model"]["rollout"]["name"] = None
    tree = _resolve_env(tree, os.environ if environ is None else environ)
    if validate and experiment.family != "speedrun":
        validate_science(experiment, tree)
    missing = _find_missing(tree)
    if missing:
        raise ValueError(f"missing mandatory value(s): {', '.join(missing)}")
    return tree


def validate_science(experiment: Experiment, config: dict) -> None:
    """Fail-closed invariants of the agentic RL pilots (reference :149-229); each message names the
    violated rule.  The MFU device name must say which accelerator the job really runs on: B200."""
    c = Tree(config)
    actor, rollout = c.actor_rollout_ref.actor, c.actor_rollout_ref.rollout
    strategy = "fsdp2" if experiment.engine == "dp" else "megatron"
    if c.model_engine != experiment.engine or actor.strategy != strategy:
        raise ValueError("resolved learner strategy differs from the experiment engine")
    if c.algorithm.adv_estimator != "grpo":
        raise ValueError("the agentic code pilot requires GRPO")
    if experiment.family == "muse_glimmer":
        _validate_muse_science(experiment, c)
    elif experiment.engine == "megatron":
        if actor.megatron.dtype != "bfloat16":
            raise ValueError("native mixed precision requires the bfloat16 Megatron contract")
        if actor.megatron.patch_recomputation_backward:
            raise ValueError("native Limite owns checkpointing; runtime Megatron patches must be disabled")
    if experiment.family == "limite" and c.actor_rollout_ref.model.override_config:
        raise ValueError("model geometry overrides require a new verified export")
    if experiment.intervention == "replace_attention":
        _validate_conversion_science(experiment, c)
    if experiment.family == "limite" and not rollout.enforce_eager:
        comp = rollout.engine_kwargs.vllm.get("compilation_config", {}) or {}
        if (rollout.max_num_seqs != 1 or comp.get("mode") != 0 or comp.get("cudagraph_mode") != "FULL_DECODE_ONLY"
                or comp.get("cudagraph_capture_sizes") != [1] or comp.get("max_cudagraph_capture_size") != 1):
            raise ValueError("native serving requires eager execution or explicit single-sequence decode graphs")
    if experiment.family == "limite" and experiment.attention == "native":
        att = rollout.engine_kwargs.vllm.attention_config
        if experiment.variant != "normal" or att.backend != "FLASH_ATTN" or att.flash_attn_version != 2:
            raise ValueError("native normal RL requires explicit FlashAttention-2 serving")
    if rollout.checkpoint_engine.backend != "naive":
        raise ValueError("native mixed precision requires qualified full-weight synchronization")
    if rollout.max_model_len != experiment.native_context:
        raise ValueError("rollout must retain the model's native context")
    if rollout.prompt_length + rollout.response_length != experiment.native_context:
        raise ValueError("prompt and response allocation must cover native context")
    if c.data.max_prompt_length != rollout.prompt_length or c.data.max_response_length != rollout.response_length:
        raise ValueError("dataset and agent context geometry differ")
    if c.data.truncation != "error":
        raise ValueError("silently truncating agentic task prompts is not allowed")
    if not rollout.multi_turn.enable or not rollout.calculate_log_probs:
        raise ValueError("agentic RL requires multi-turn rollout and behavior log probabilities")
    if rollout.n < 2:
        raise ValueError("GRPO requires multiple responses and recorded behavior probabilities")
    cor = c.algorithm.rollout_correction
    if cor.bypass_mode or cor.rollout_is != "token" or cor.rollout_is_threshold != 2.0 or cor.rollout_is_batch_normalize:
        raise ValueError("the pilot requires one upstream token importance correction, capped at 2")
    if actor.use_kl_loss or c.algorithm.use_kl_in_reward:
        raise ValueError("this controlled code pilot does not include a reference-policy KL")
    if (experiment.family == "limite" and experiment.intervention != "replace_attention"
            and rollout.custom.agent_framework.mask_unfinished_episode):
        raise ValueError("unfinished trajectories must remain visible in this pilot")
    if not 0 <= c.trainer.v1.sampler.max_off_policy_threshold <= experiment.maximum_policy_lag:
        raise ValueError("policy lag exceeds the explicit experiment contract")
    if experiment.resume_checkpoint:
        if c.trainer.resume_mode != "resume_path" or c.trainer.resume_from_path != experiment.resume_checkpoint:
            raise ValueError("resume must use the explicit checkpoint lineage")
    elif c.trainer.resume_mode != "disable":
        raise ValueError("fresh RL must reset the optimizer, RNG and training counters")
    if (rollout.custom.agent_framework.get("trajectory_validator") != "archlab_b200.train.rollout.RolloutContract"
            or c.trainer.get("metrics_extension") != "archlab_b200.train.metrics.step_metrics"):
        raise ValueError("the primary pilot requires validated rollout and performance contracts")
    if c.ray_kwargs.ray_init.runtime_env.env_vars.get("VERL_MFU_DEVICE_NAME") != "B200":
        raise ValueError("MFU hardware must reflect the actual B200 allocation")
    if experiment.family == "qwen3_5":
        model = c.actor_rollout_ref.model
        if (model.path != experiment.parent_checkpoint or model.external_lib or model.trust_remote_code
                or model.custom_chat_template
                or dict(model.override_config) != {"attn_implementation": "flash_attention_2"}
                or dict(c.data.apply_chat_template_kwargs) != {"enable_thinking": False}
                or actor.fsdp_config.dtype != "bfloat16" or actor.fsdp_config.model_dtype != "fp32"
                or rollout.multi_turn.format != "qwen3_coder" or rollout.logprobs_mode != "processed_logprobs"):
            raise ValueError("Qwen native control requires its declared model, codec and mixed precision")


def _validate_muse_science(e: Experiment, c: Tree) -> None:
    actor, model, rollout = c.actor_rollout_ref.actor, c.actor_rollout_ref.model, c.actor_rollout_ref.rollout
    if (model.path != e.parent_checkpoint or model.external_lib or model.trust_remote_code
            or model.custom_chat_template or model.hf_config_path or model.tokenizer_path):
        raise ValueError("Muse must load its unchanged publisher checkpoint, tokenizer and template together")
    if dict(model.override_config) != {"attn_implementation": "flash_attention_4"}:
        raise ValueError("Muse permits only its explicit native FlashAttention-4 kernel override, without geometry changes")
    f = actor.fsdp_config
    if (f.strategy != "fsdp2" or f.dtype != "bfloat16" or f.model_dtype != "fp32" or f.ulysses_sequence_parallel_size != 1
            or f.fsdp_size != 8 or f.param_offload or f.optimizer_offload or c.trainer.nnodes != 1
            or c.trainer.n_gpus_per_node != 8):
        raise ValueError("Muse requires GPU-resident DP8 FSDP2 with FP32 master weights and BF16 compute")
    if (model.use_remove_padding or model.use_fused_kernels or model.use_liger or model.lora_rank or model.lora.rank
            or model.lora_adapter_path or not model.enable_gradient_checkpointing or model.mtp.enable
            or actor.ppo_micro_batch_size_per_gpu != 1 or actor.use_dynamic_bsz or actor.use_torch_compile
            or f.use_torch_compile or f.qat.enable):
        raise ValueError("Muse admission requires native full-weight microbatches without unqualified kernels or quantization")
    o = actor.optim
    if (o.optimizer != "Adam" or o.optimizer_impl != "torch.optim" or o.lr != 1e-6 or list(o.betas) != [.9, .95]
            or o.weight_decay != 0 or o.override_optimizer_config):
        raise ValueError("Muse control requires explicit torch Adam at 1e-6 with betas (0.9, 0.95)")
    if (e.execution != "colocate_async" or e.native_context != 131072 or rollout.name != "vllm"
            or not rollout.enforce_eager or rollout.ignore_eos or rollout.prompt_length != 16384
            or rollout.response_length != 114688 or rollout.quantization or rollout.quantization_config_file
            or rollout.tensor_model_parallel_size != 1 or rollout.pipeline_model_parallel_size != 1
            or rollout.data_parallel_size != 1 or rollout.max_num_seqs != 1 or rollout.gpu_memory_utilization != .3
            or rollout.multi_turn.format != "muse_glimmer"
            or dict(rollout.engine_kwargs.vllm) != {"model_impl": "vllm", "limit_mm_per_prompt": {"image": 0, "video": 0}}
            or dict(c.data.apply_chat_template_kwargs) != {"reasoning_strength": "high"}):
        raise ValueError("Muse control requires native eager vLLM serving and the publisher's reasoning/tool protocol")
    v = rollout.val_kwargs
    if (rollout.temperature != 1. or not rollout.do_sample or rollout.top_p != 1. or rollout.top_k != -1
            or rollout.logprobs_mode != "processed_logprobs" or not v.do_sample
            or any(v[k] != rollout[k] for k in ("temperature", "top_p", "top_k"))):
        raise ValueError("Muse control requires full-support processed behavior probabilities")
    if (c.data.train_batch_size != 2 or actor.ppo_mini_batch_size != 2 or rollout.n != 4
            or c.algorithm.filter_groups.enable or not c.algorithm.norm_adv_by_std_in_grpo
            or not rollout.custom.agent_framework.mask_unfinished_episode):
        raise ValueError("Muse control requires two stock GRPO groups of four and unfinished-episode masking")
    p = e.pilot
    if (p is None or p.max_turn_tokens != 8192 or p.step_limit != 500 or p.minimum_prompt_groups != 2
            or p.minimum_completed_verifiers != 8
            or min(p.minimum_tool_calls, p.minimum_observation_tokens, p.minimum_reward_contrast_groups) < 1
            or p.maximum_truncated_trajectories != 0):
        raise ValueError("Muse admission requires complete agentic traces, executable rewards and reward contrast")


def _validate_conversion_science(e: Experiment, c: Tree) -> None:
    actor, model, rollout = c.actor_rollout_ref.actor, c.actor_rollout_ref.model, c.actor_rollout_ref.rollout
    t = rollout.temperature
    if (type(t) not in (float, int) or not math.isfinite(t) or t <= 0 or not rollout.do_sample
            or rollout.top_p != 1. or rollout.top_k != -1 or rollout.logprobs_mode != "processed_logprobs"):
        raise ValueError("replacement RL requires positive-temperature full-support processed behavior probabilities")
    v = rollout.val_kwargs
    if not v.do_sample or any(v[k] != rollout[k] for k in ("temperature", "top_p", "top_k")):
        raise ValueError("replacement validation and training must use the declared harness sampling distribution")
    if (e.parent_stage != "package_sft" or e.parent_tokens is not None or e.variant != "simplicial"
            or e.attention != "tilelang" or e.execution != "colocate_async"):
        raise ValueError("replacement RL requires package SFT lineage and bounded async TileLang execution")
    mg = actor.megatron
    if (model.external_lib != "archlab_b200.train.learner" or model.use_remove_padding or model.use_fused_kernels
            or model.lora_rank or model.lora.rank or mg.use_remove_padding or mg.pad_bshd_to_minibatch_max
            or actor.ppo_micro_batch_size_per_gpu != 1 or actor.use_dynamic_bsz):
        raise ValueError("replacement RL requires full-weight native BSHD microbatches of one")
    if (any(mg[n] != 1 for n in ("tensor_model_parallel_size", "pipeline_model_parallel_size",
                                 "context_parallel_size", "expert_model_parallel_size"))
            or mg.sequence_parallel or mg.dynamic_context_parallel
            or mg.virtual_pipeline_model_parallel_size is not None or c.trainer.nnodes != 1
            or c.trainer.n_gpus_per_node != 8):
        raise ValueError("replacement learner requires DP8 with TP=PP=CP=EP=1")
    att = rollout.engine_kwargs.vllm.attention_config
    if (rollout.name != "vllm" or not rollout.enforce_eager or rollout.max_num_seqs != 1
            or rollout.enable_prefix_caching or rollout.enable_chunked_prefill
            or rollout.max_num_batched_tokens < e.native_context or rollout.tensor_model_parallel_size != 1
            or rollout.pipeline_model_parallel_size != 1 or rollout.data_parallel_size != 1
            or att.backend != "FLASH_ATTN" or att.flash_attn_version != 2):
        raise ValueError("replacement serving requires eager FA2, one request, TP=PP=1 and no prefix/chunked prefill")
    conflicting = {"enforce_eager", "max_num_seqs", "enable_prefix_caching", "enable_chunked_prefill",
                   "tensor_parallel_size", "pipeline_parallel_size", "decode_context_parallel_size",
                   "prefill_context_parallel_size", "quantization", "kv_cache_dtype", "speculative_config",
                   "hf_overrides", "model", "logprobs_mode"} & set(rollout.engine_kwargs.vllm)
    if conflicting:
        raise ValueError("replacement engine kwargs override the serving contract: " + ", ".join(sorted(conflicting)))
    if not actor.optim.use_checkpoint_opt_param_scheduler:
        raise ValueError("replacement checkpoints must restore the optimizer parameter scheduler")
    ov = actor.optim.override_optimizer_config or {}
    if ov.get("adam_beta1") != .9 or ov.get("adam_beta2") != .95:
        raise ValueError("replacement Adam requires explicit Megatron beta overrides (0.9, 0.95)")
    p = e.pilot
    if (p is None or not 0 < p.max_turn_tokens <= 8192 or p.step_limit != 500 or p.minimum_prompt_groups < 2
            or p.minimum_completed_verifiers < p.minimum_prompt_groups * rollout.n
            or min(p.minimum_tool_calls, p.minimum_observation_tokens, p.minimum_reward_contrast_groups) < 1
            or p.maximum_truncated_trajectories != 0 or c.data.train_batch_size < p.minimum_prompt_groups
            or actor.ppo_mini_batch_size * rollout.n < 8 or not rollout.custom.agent_framework.mask_unfinished_episode):
        raise ValueError("replacement pilot requires explicit short turns, usable traces and stock truncation masking")
