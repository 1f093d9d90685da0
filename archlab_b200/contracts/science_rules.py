"""The fail-closed science rules of the agentic RL pilots, as a table.

A rule is a message, a condition on the experiment that says when it applies, and a set of *pins*: dotted paths into the
resolved trainer tree (or ``e.<field>`` for the experiment itself) with the value each must have.  A pin's requirement is
a literal (equality), ``ON`` / ``OFF`` (truthy / falsy), or a function ``(value, experiment, tree) -> bool``.  The first
rule with a violated pin raises ``ValueError(rule.message)``; the messages are the contract the reference's validators
expose (src/archlab/training/config.py:149-229, :232-330), the evaluation scheme is this file's.

Path shorthands: ``actor.``, ``rollout.``, ``model.`` live under ``actor_rollout_ref``; ``mg.`` is ``actor.megatron``;
``fsdp.`` is ``actor.fsdp_config``; ``vllm.`` is ``rollout.engine_kwargs.vllm``; ``agent.`` is
``rollout.custom.agent_framework``; ``pilot.`` is the experiment's pilot thresholds.  A path ending in ``?`` may be absent
(its value is then ``None``); any other missing path violates the rule.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Callable

ON, OFF = object(), object()
_ABSENT = object()
_SHORT = {"actor": "actor_rollout_ref.actor", "rollout": "actor_rollout_ref.rollout", "model": "actor_rollout_ref.model",
          "mg": "actor_rollout_ref.actor.megatron", "fsdp": "actor_rollout_ref.actor.fsdp_config",
          "vllm": "actor_rollout_ref.rollout.engine_kwargs.vllm", "agent": "actor_rollout_ref.rollout.custom.agent_framework"}


def lookup(tree: dict, experiment, path: str) -> Any:
    optional = path.endswith("?")
    head, _, rest = path.rstrip("?").partition(".")
    if head == "e":
        return getattr(experiment, rest)
    if head == "pilot":
        return getattr(experiment.pilot, rest, _ABSENT) if experiment.pilot is not None else _ABSENT
    node: Any = tree
    full = path.rstrip("?") if head not in _SHORT else _SHORT[head] + (f".{rest}" if rest else "")
    for key in full.split("."):
        if not isinstance(node, dict) or key not in node:
            return None if optional else _ABSENT
        node = node[key]
    return node


def _plain(value: Any) -> Any:
    return {k: _plain(v) for k, v in value.items()} if isinstance(value, dict) else list(value) if isinstance(value, (list, tuple)) else value


@dataclass(frozen=True)
class Rule:
    message: str
    pins: dict[str, Any]
    when: Callable[[Any], bool] = field(default=lambda e: True)

    def violated(self, experiment, tree: dict) -> str | None:
        for path, want in self.pins.items():
            got = lookup(tree, experiment, path)
            if got is _ABSENT:
                return path
            ok = bool(got) if want is ON else not got if want is OFF else want(got, experiment, tree) if callable(want) \
                else _plain(got) == want
            if not ok:
                return path
        return None


def check(rules, experiment, tree: dict) -> None:
    for rule in rules:
        if rule.when(experiment) and (path := rule.violated(experiment, tree)) is not None:
            error = ValueError(rule.message)
            error.violated_path = path
            raise error


# ---- requirement helpers ---------------------------------------------------------------------------------------------
def same_as(path: str):
    return lambda got, e, tree: got == lookup(tree, e, path)


def at_least(bound):
    return lambda got, e, tree: got >= (bound(e, tree) if callable(bound) else bound)


def _rollout_n(e, tree):
    return lookup(tree, e, "rollout.n")


_positive_finite = lambda t, e, tree: type(t) in (float, int) and math.isfinite(t) and t > 0
_is = lambda **fields: (lambda e: all(getattr(e, k) == v for k, v in fields.items()))
_FULL_SUPPORT = {"rollout.do_sample": ON, "rollout.top_p": 1.0, "rollout.top_k": -1, "rollout.logprobs_mode": "processed_logprobs"}
_VALIDATION_SAMPLES_LIKE_TRAINING = {"rollout.val_kwargs.do_sample": ON, "rollout.val_kwargs.temperature": same_as("rollout.temperature"),
                                     "rollout.val_kwargs.top_p": same_as("rollout.top_p"), "rollout.val_kwargs.top_k": same_as("rollout.top_k")}
_PILOT_FLOORS = {f"pilot.minimum_{k}": at_least(1) for k in ("tool_calls", "observation_tokens", "reward_contrast_groups")}
_SERVING_KEYS_OWNED_BY_THE_CONTRACT = frozenset({
    "enforce_eager", "max_num_seqs", "enable_prefix_caching", "enable_chunked_prefill", "tensor_parallel_size", "pipeline_parallel_size",
    "decode_context_parallel_size", "prefill_context_parallel_size", "quantization", "kv_cache_dtype", "speculative_config",
    "hf_overrides", "model", "logprobs_mode"})

MUSE = (
    Rule("Muse must load its unchanged publisher checkpoint, tokenizer and template together",
         {"model.path": same_as("e.parent_checkpoint"), "model.external_lib": OFF, "model.trust_remote_code": OFF,
          "model.custom_chat_template": OFF, "model.hf_config_path": OFF, "model.tokenizer_path": OFF}),
    Rule("Muse permits only its explicit native FlashAttention-4 kernel override, without geometry changes",
         {"model.override_config": {"attn_implementation": "flash_attention_4"}}),
    Rule("Muse requires GPU-resident DP8 FSDP2 with FP32 master weights and BF16 compute",
         {"fsdp.strategy": "fsdp2", "fsdp.dtype": "bfloat16", "fsdp.model_dtype": "fp32", "fsdp.ulysses_sequence_parallel_size": 1,
          "fsdp.fsdp_size": 8, "fsdp.param_offload": OFF, "fsdp.optimizer_offload": OFF, "trainer.nnodes": 1, "trainer.n_gpus_per_node": 8}),
    Rule("Muse admission requires native full-weight microbatches without unqualified kernels or quantization",
         {"model.use_remove_padding": OFF, "model.use_fused_kernels": OFF, "model.use_liger": OFF, "model.lora_rank": OFF,
          "model.lora.rank": OFF, "model.lora_adapter_path": OFF, "model.enable_gradient_checkpointing": ON, "model.mtp.enable": OFF,
          "actor.ppo_micro_batch_size_per_gpu": 1, "actor.use_dynamic_bsz": OFF, "actor.use_torch_compile": OFF,
          "fsdp.use_torch_compile": OFF, "fsdp.qat.enable": OFF}),
    Rule("Muse control requires explicit torch Adam at 1e-6 with betas (0.9, 0.95)",
         {"actor.optim.optimizer": "Adam", "actor.optim.optimizer_impl": "torch.optim", "actor.optim.lr": 1e-6,
          "actor.optim.betas": [0.9, 0.95], "actor.optim.weight_decay": 0, "actor.optim.override_optimizer_config": OFF}),
    Rule("Muse control requires native eager vLLM serving and the publisher's reasoning/tool protocol",
         {"e.execution": "colocate_async", "e.native_context": 131072, "rollout.name": "vllm", "rollout.enforce_eager": ON,
          "rollout.ignore_eos": OFF, "rollout.prompt_length": 16384, "rollout.response_length": 114688, "rollout.quantization": OFF,
          "rollout.quantization_config_file": OFF, "rollout.tensor_model_parallel_size": 1, "rollout.pipeline_model_parallel_size": 1,
          "rollout.data_parallel_size": 1, "rollout.max_num_seqs": 1, "rollout.gpu_memory_utilization": 0.3,
          "rollout.multi_turn.format": "muse_glimmer",
          "vllm": {"model_impl": "vllm", "limit_mm_per_prompt": {"image": 0, "video": 0}},
          "data.apply_chat_template_kwargs": {"reasoning_strength": "high"}}),
    Rule("Muse control requires full-support processed behavior probabilities",
         {"rollout.temperature": 1.0, **_FULL_SUPPORT, **_VALIDATION_SAMPLES_LIKE_TRAINING}),
    Rule("Muse control requires two stock GRPO groups of four and unfinished-episode masking",
         {"data.train_batch_size": 2, "actor.ppo_mini_batch_size": 2, "rollout.n": 4, "algorithm.filter_groups.enable": OFF,
          "algorithm.norm_adv_by_std_in_grpo": ON, "agent.mask_unfinished_episode": ON}),
    Rule("Muse admission requires complete agentic traces, executable rewards and reward contrast",
         {"pilot.max_turn_tokens": 8192, "pilot.step_limit": 500, "pilot.minimum_prompt_groups": 2, "pilot.minimum_completed_verifiers": 8,
          **_PILOT_FLOORS, "pilot.maximum_truncated_trajectories": 0}),
)

CONVERSION = (
    Rule("replacement RL requires positive-temperature full-support processed behavior probabilities",
         {"rollout.temperature": _positive_finite, **_FULL_SUPPORT}),
    Rule("replacement validation and training must use the declared harness sampling distribution", _VALIDATION_SAMPLES_LIKE_TRAINING),
    Rule("replacement RL requires package SFT lineage and bounded async TileLang execution",
         {"e.parent_stage": "package_sft", "e.parent_tokens": None, "e.variant": "simplicial", "e.attention": "tilelang",
          "e.execution": "colocate_async"}),
    Rule("replacement RL requires full-weight native BSHD microbatches of one",
         {"model.external_lib": "archlab_b200.train.learner", "model.use_remove_padding": OFF, "model.use_fused_kernels": OFF,
          "model.lora_rank": OFF, "model.lora.rank": OFF, "mg.use_remove_padding": OFF, "mg.pad_bshd_to_minibatch_max": OFF,
          "actor.ppo_micro_batch_size_per_gpu": 1, "actor.use_dynamic_bsz": OFF}),
    Rule("replacement learner requires DP8 with TP=PP=CP=EP=1",
         {"mg.tensor_model_parallel_size": 1, "mg.pipeline_model_parallel_size": 1, "mg.context_parallel_size": 1,
          "mg.expert_model_parallel_size": 1, "mg.sequence_parallel": OFF, "mg.dynamic_context_parallel": OFF,
          "mg.virtual_pipeline_model_parallel_size": None, "trainer.nnodes": 1, "trainer.n_gpus_per_node": 8}),
    Rule("replacement serving requires eager FA2, one request, TP=PP=1 and no prefix/chunked prefill",
         {"rollout.name": "vllm", "rollout.enforce_eager": ON, "rollout.max_num_seqs": 1, "rollout.enable_prefix_caching": OFF,
          "rollout.enable_chunked_prefill": OFF, "rollout.max_num_batched_tokens": at_least(lambda e, tree: e.native_context),
          "rollout.tensor_model_parallel_size": 1, "rollout.pipeline_model_parallel_size": 1, "rollout.data_parallel_size": 1,
          "vllm.attention_config.backend": "FLASH_ATTN", "vllm.attention_config.flash_attn_version": 2}),
    # (the engine-kwargs rule names the offending keys; see ``conversion_kwargs_conflict``)
    Rule("replacement checkpoints must restore the optimizer parameter scheduler", {"actor.optim.use_checkpoint_opt_param_scheduler": ON}),
    Rule("replacement Adam requires explicit Megatron beta overrides (0.9, 0.95)",
         {"actor.optim.override_optimizer_config?": lambda ov, e, tree: (ov or {}).get("adam_beta1") == 0.9 and (ov or {}).get("adam_beta2") == 0.95}),
    Rule("replacement pilot requires explicit short turns, usable traces and stock truncation masking",
         {"pilot.max_turn_tokens": lambda v, e, tree: 0 < v <= 8192, "pilot.step_limit": 500, "pilot.minimum_prompt_groups": at_least(2),
          "pilot.minimum_completed_verifiers": at_least(lambda e, tree: e.pilot.minimum_prompt_groups * _rollout_n(e, tree)),
          **_PILOT_FLOORS, "pilot.maximum_truncated_trajectories": 0,
          "data.train_batch_size": at_least(lambda e, tree: e.pilot.minimum_prompt_groups),
          "actor.ppo_mini_batch_size": lambda v, e, tree: v * _rollout_n(e, tree) >= 8, "agent.mask_unfinished_episode": ON}),
)
_CONVERSION_KWARGS_AFTER = "replacement serving requires eager FA2, one request, TP=PP=1 and no prefix/chunked prefill"


def conversion_kwargs_conflict(experiment, tree: dict) -> None:
    taken = _SERVING_KEYS_OWNED_BY_THE_CONTRACT & set(lookup(tree, experiment, "vllm") or {})
    if taken:
        raise ValueError("replacement engine kwargs override the serving contract: " + ", ".join(sorted(taken)))


_limite, _megatron_not_muse = _is(family="limite"), lambda e: e.engine == "megatron" and e.family != "muse_glimmer"
_single_sequence_graphs = {"mode": 0, "cudagraph_mode": "FULL_DECODE_ONLY", "cudagraph_capture_sizes": [1], "max_cudagraph_capture_size": 1}

HEAD = (
    Rule("resolved learner strategy differs from the experiment engine",
         {"model_engine": same_as("e.engine"), "actor.strategy": lambda got, e, tree: got == ("fsdp2" if e.engine == "dp" else "megatron")}),
    Rule("the agentic code pilot requires GRPO", {"algorithm.adv_estimator": "grpo"}),
)
FAMILY = (
    Rule("native mixed precision requires the bfloat16 Megatron contract", {"mg.dtype": "bfloat16"}, _megatron_not_muse),
    Rule("native Limite owns checkpointing; runtime Megatron patches must be disabled", {"mg.patch_recomputation_backward": OFF}, _megatron_not_muse),
    Rule("model geometry overrides require a new verified export", {"model.override_config": OFF}, _limite),
)
COMMON = (
    Rule("native normal RL requires explicit FlashAttention-2 serving",
         {"e.variant": "normal", "vllm.attention_config.backend": "FLASH_ATTN", "vllm.attention_config.flash_attn_version": 2},
         _is(family="limite", attention="native")),
    Rule("native mixed precision requires qualified full-weight synchronization", {"rollout.checkpoint_engine.backend": "naive"}),
    Rule("rollout must retain the model's native context", {"rollout.max_model_len": same_as("e.native_context")}),
    Rule("prompt and response allocation must cover native context",
         {"rollout.prompt_length": lambda p, e, tree: p + lookup(tree, e, "rollout.response_length") == e.native_context}),
    Rule("dataset and agent context geometry differ",
         {"data.max_prompt_length": same_as("rollout.prompt_length"), "data.max_response_length": same_as("rollout.response_length")}),
    Rule("silently truncating agentic task prompts is not allowed", {"data.truncation": "error"}),
    Rule("agentic RL requires multi-turn rollout and behavior log probabilities",
         {"rollout.multi_turn.enable": ON, "rollout.calculate_log_probs": ON}),
    Rule("GRPO requires multiple responses and recorded behavior probabilities", {"rollout.n": at_least(2)}),
    Rule("the pilot requires one upstream token importance correction, capped at 2",
         {"algorithm.rollout_correction.bypass_mode": OFF, "algorithm.rollout_correction.rollout_is": "token",
          "algorithm.rollout_correction.rollout_is_threshold": 2.0, "algorithm.rollout_correction.rollout_is_batch_normalize": OFF}),
    Rule("this controlled code pilot does not include a reference-policy KL", {"actor.use_kl_loss": OFF, "algorithm.use_kl_in_reward": OFF}),
    Rule("unfinished trajectories must remain visible in this pilot", {"agent.mask_unfinished_episode": OFF},
         lambda e: e.family == "limite" and e.intervention != "replace_attention"),
    Rule("policy lag exceeds the explicit experiment contract",
         {"trainer.v1.sampler.max_off_policy_threshold": lambda lag, e, tree: 0 <= lag <= e.maximum_policy_lag}),
    Rule("resume must use the explicit checkpoint lineage",
         {"trainer.resume_mode": "resume_path", "trainer.resume_from_path": same_as("e.resume_checkpoint")}, lambda e: bool(e.resume_checkpoint)),
    Rule("fresh RL must reset the optimizer, RNG and training counters", {"trainer.resume_mode": "disable"}, lambda e: not e.resume_checkpoint),
    Rule("the primary pilot requires validated rollout and performance contracts",
         {"agent.trajectory_validator?": "archlab_b200.train.rollout.RolloutContract",
          "trainer.metrics_extension?": "archlab_b200.train.metrics.step_metrics"}),
    # the MFU accounting must name the accelerator the job really runs on
    Rule("MFU hardware must reflect the actual B200 allocation", {"ray_kwargs.ray_init.runtime_env.env_vars.VERL_MFU_DEVICE_NAME?": "B200"}),
    Rule("Qwen native control requires its declared model, codec and mixed precision",
         {"model.path": same_as("e.parent_checkpoint"), "model.external_lib": OFF, "model.trust_remote_code": OFF,
          "model.custom_chat_template": OFF, "model.override_config": {"attn_implementation": "flash_attention_2"},
          "data.apply_chat_template_kwargs": {"enable_thinking": False}, "fsdp.dtype": "bfloat16", "fsdp.model_dtype": "fp32",
          "rollout.multi_turn.format": "qwen3_coder", "rollout.logprobs_mode": "processed_logprobs"}, _is(family="qwen3_5")),
)


def _graph_serving(experiment, tree: dict) -> None:
    """Limite serving without eager mode must pin single-sequence decode graphs."""
    if experiment.family != "limite" or lookup(tree, experiment, "rollout.enforce_eager"):
        return
    compilation = lookup(tree, experiment, "vllm.compilation_config?") or {}
    pinned = lookup(tree, experiment, "rollout.max_num_seqs") == 1 and all(_plain(compilation.get(k)) == v for k, v in _single_sequence_graphs.items())
    if not pinned:
        raise ValueError("native serving requires eager execution or explicit single-sequence decode graphs")


def validate(experiment, tree: dict) -> None:
    check(HEAD, experiment, tree)
    if experiment.family == "muse_glimmer":
        check(MUSE, experiment, tree)
    check(FAMILY, experiment, tree)
    if experiment.intervention == "replace_attention":
        split = next(i for i, r in enumerate(CONVERSION) if r.message == _CONVERSION_KWARGS_AFTER) + 1
        check(CONVERSION[:split], experiment, tree)
        conversion_kwargs_conflict(experiment, tree)
        check(CONVERSION[split:], experiment, tree)
    _graph_serving(experiment, tree)
    check(COMMON, experiment, tree)
