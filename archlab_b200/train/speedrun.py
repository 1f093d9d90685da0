"""Speedrun trainer: one object that owns model, engine, optimizer and the step protocol.

The public call is ``Trainer.train_step(tokens)`` where ``tokens`` is a pinned host tensor
``[local_batch, T + 1]`` of int64 ids (inputs are ``[:, :-1]``, labels ``[:, 1:]``).  One call does
what one iteration of the reference's loop does (src/archlab/speedrun/base_train.py:1812-1870):
host->device copy, gradient accumulation over micro-batches, schedule, optimizer step (gradient
synchronisation lives inside the optimizer, as in the reference), and returns the mean loss as a
Python float (a device->host read).

On CUDA the model runs through ``FusedGPTEngine``; on CPU (gloo tests, tiny configs) through the
eager module with autograd.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..models.nanochat import GPT, GPTConfig
from ..optim.setup import Schedule, setup_model_optimizer
from ..parallel import collectives as coll


@dataclass
class TrainerConfig:
    model: GPTConfig
    micro_batch: int = 8            # sequences per forward/backward
    num_iterations: int = 1000
    matrix_lr: float = 0.02
    embedding_lr: float = 0.2
    unembedding_lr: float = 0.004
    scalar_lr: float = 0.5
    weight_decay: float = 0.0
    matrix_optimizer: str = "normuon"
    warmup_steps: int = 40
    warmdown_ratio: float = 0.65
    final_lr_frac: float = 0.05
    seed: int = 0
    head_chunk: int = 8192
    zero_impl: str = "auto"         # "nccl" (decomposed baseline) | "fused" (peer-memory kernels) | "auto"
    use_engine: bool = True         # False: module forward + autograd on CUDA too (the library-kernel baseline)


class Trainer:
    def __init__(self, cfg: TrainerConfig, device: torch.device | str = "cpu"):
        self.cfg = cfg
        self.device = torch.device(device)
        torch.manual_seed(cfg.seed)
        with torch.device("meta"):
            model = GPT(cfg.model)
        model.to_empty(device=self.device)
        model.init_weights()
        self.model = model
        self.engine = None
        if self.device.type == "cuda" and cfg.use_engine and cfg.model.head_dim == 128:
            from ..models.nanochat_engine import FusedGPTEngine

            ws = coll.world_size()
            self.use_peer = ws > 1 and cfg.zero_impl in ("auto", "fused") and cfg.matrix_optimizer == "normuon"
            self.engine = FusedGPTEngine(model, head_chunk=cfg.head_chunk, world=ws, symmetric=self.use_peer)
        self.world = coll.world_size()
        if self.world > 1:
            # identical parameters on every rank (seeded init makes them equal already; this is the
            # cross-replica equality the reference asserts before training)
            for p in model.parameters():
                dist.broadcast(p.data, src=0)
            if self.engine is not None:
                self.engine.refresh_shadows()
        if self.engine is not None and cfg.matrix_optimizer == "normuon":
            from ..optim.fused import FusedMuonAdamW
            from ..optim.fused_peer import PeerMuonAdamW

            self.optimizer = (PeerMuonAdamW if self.use_peer else FusedMuonAdamW)(
                model, self.engine.store, unembedding_lr=cfg.unembedding_lr, embedding_lr=cfg.embedding_lr,
                matrix_lr=cfg.matrix_lr, weight_decay=cfg.weight_decay, scalar_lr=cfg.scalar_lr)
            self.fused_optimizer = True
        else:
            self.fused_optimizer = False
            self.optimizer = setup_model_optimizer(
                model, unembedding_lr=cfg.unembedding_lr, embedding_lr=cfg.embedding_lr, matrix_lr=cfg.matrix_lr,
                weight_decay=cfg.weight_decay, scalar_lr=cfg.scalar_lr, matrix_optimizer=cfg.matrix_optimizer,
                distributed=self.world > 1)
        self.schedule = Schedule(cfg.num_iterations, cfg.warmup_steps, cfg.warmdown_ratio, cfg.final_lr_frac,
                                 cfg.weight_decay)
        self.step_index = 0
        self._dev_tokens = None

    # ------------------------------------------------------------------
    def _to_device(self, tokens: torch.Tensor) -> torch.Tensor:
        if self.device.type != "cuda":
            return tokens
        if self._dev_tokens is None or self._dev_tokens.shape != tokens.shape:
            self._dev_tokens = torch.empty(tokens.shape, dtype=tokens.dtype, device=self.device)
        self._dev_tokens.copy_(tokens, non_blocking=True)
        return self._dev_tokens

    def train_step_device(self, tok: torch.Tensor) -> torch.Tensor:
        """One optimizer step on a token block already resident on the device; returns the mean
        loss as a 0-d device tensor (no host synchronisation)."""
        cfg = self.cfg
        x, y = tok[:, :-1], tok[:, 1:]
        nb = x.size(0)
        mb = min(cfg.micro_batch, nb)
        if nb % mb:
            raise ValueError("local batch must be a multiple of the micro batch")
        n_valid = float(y.numel())     # synthetic / packed data has no ignored labels
        if self.engine is not None:
            self.engine.store.zero_grads()
            loss_sum = None
            for s in range(0, nb, mb):
                ls = self.engine.forward_backward(x[s:s + mb].contiguous(), y[s:s + mb].contiguous(),
                                                  1.0 / n_valid)
                loss_sum = ls if loss_sum is None else loss_sum + ls
            self.engine.finish_step()
        else:
            self.model.train()
            self.model.zero_grad(set_to_none=True)
            loss_sum = None
            for s in range(0, nb, mb):
                ls = self.model(x[s:s + mb], y[s:s + mb], loss_reduction="sum")
                (ls / n_valid).backward()
                loss_sum = ls.detach() if loss_sum is None else loss_sum + ls.detach()
        self.schedule.apply(self.optimizer, self.step_index)
        self.optimizer.step()
        if self.engine is not None and not self.fused_optimizer:
            self.engine.refresh_shadows()   # the fused optimizer writes the bf16 shadows itself
        self.step_index += 1
        return loss_sum / n_valid

    def train_step(self, tokens: torch.Tensor) -> float:
        """One optimizer step on this rank's ``[local_batch, T+1]`` host token block (pinned memory
        makes the copy asynchronous); returns the mean loss as a Python float."""
        return float(self.train_step_device(self._to_device(tokens)).item())

    # ------------------------------------------------------------------
    def tokens_per_step(self, local_batch: int) -> int:
        return local_batch * self.cfg.model.sequence_len * self.world
