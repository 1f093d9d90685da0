"""Per-step RL metrics callback and MFU bookkeeping (src/archlab/training/metrics.py:9-77).

``allocated_gpu_seconds`` is phase time multiplied by the number of allocated GPUs - it is NOT
measured idleness (colocated GPUs generate while the learner waits).  The reference constant for
MFU is the measured/nominal dense bf16 throughput of a B200.
"""
from __future__ import annotations

import math
from collections import defaultdict

B200_DENSE_BF16_FLOPS = 2.25e15       # nominal dense peak; measured roofline lives in MEASURED_PEAKS.json
PHASES = ("gen", "reward", "old_log_prob", "ref", "values", "adv", "update_critic", "update_actor",
          "save_checkpoint", "update_weights")


def _get(node, dotted: str):
    for part in dotted.split("."):
        node = node[part] if isinstance(node, dict) else getattr(node, part)
    return node


def step_metrics(*, config, batch, tags, timing, step) -> dict:
    if _get(config, "trainer.v1.trainer_mode") not in {"sync", "colocate_async"}:
        raise ValueError("phase accounting needs a resource map for separate rollout pools")
    gpus = _get(config, "trainer.nnodes") * _get(config, "trainer.n_gpus_per_node")
    seconds = float(timing["step"])
    if seconds <= 0 or any(not math.isfinite(v) or v < 0 for v in timing.values()):
        raise ValueError("invalid step timing")
    measured = sum(timing.get(k, 0) for k in PHASES)
    if measured > seconds * 1.01:
        raise ValueError("phase timers overlap; cannot report additive GPU-seconds")
    out = {f"perf/allocated_gpu_seconds/{k}": gpus * timing.get(k, 0) for k in PHASES}
    out.update({"perf/allocated_gpu_seconds/step": gpus * seconds,
                "perf/allocated_gpu_seconds/unattributed": gpus * max(0, seconds - measured),
                "perf/measured_idle_available": 0, "training/trainer_steps": step,
                "training/policy_version": step})
    masks = batch.batch["response_mask"] if hasattr(batch, "batch") else batch["response_mask"]
    scores = batch.batch["rm_scores"] if hasattr(batch, "batch") else batch["rm_scores"]
    if len(tags) != len(masks):
        raise ValueError("rollout tags and unpadded metrics batch differ")
    groups, sessions = defaultdict(list), defaultdict(set)
    for tag, reward in zip(tags, scores.sum(-1).tolist()):
        groups[tag["group_id"]].append(reward)
        sessions[tag["group_id"]].add(tag["session_id"])
    n = _get(config, "actor_rollout_ref.rollout.n")
    generated = sum(t["generated_tokens"] for t in tags)
    out.update({"rollout/consumed_generated_tokens": generated,
                "rollout/consumed_observation_tokens": sum(t["observation_tokens"] for t in tags),
                "rollout/native_eos_tokens": sum(t["native_eos_tokens"] for t in tags),
                "rollout/context_limit_count": sum(t["context_limit_reached"] for t in tags),
                "rollout/truncated_count": sum(t["termination_reason"] == "truncated" for t in tags),
                "rollout/consumed_groups": len(groups),
                "rollout/useful_groups": sum(len(set(v)) > 1 for v in groups.values()),
                "rollout/incomplete_groups": sum(len(v) != n for v in sessions.values()),
                "perf/consumed_generated_tokens_per_second": generated / seconds,
                "perf/bf16_reference_tflops_per_gpu": B200_DENSE_BF16_FLOPS / 1e12})
    return out


def model_flops_utilization(flops_per_token: float, tokens_per_second: float, n_gpus: int,
                            peak_flops: float = B200_DENSE_BF16_FLOPS) -> float:
    return flops_per_token * tokens_per_second / (n_gpus * peak_flops)
