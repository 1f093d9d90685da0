"""Mesh training entry: ``torchrun -m archlab_b200.train.mesh_train --model qwen35_4b --tp 2 ...``.

Ranks form a (pipeline, data, context, tensor) mesh with the tensor index fastest, so that a tensor
group sits on neighbouring GPUs.  Qwen3.5-family models run as ``Qwen35TP`` (tensor + sequence
parallel layers over the fused all-gather->GEMM / GEMM->reduce-scatter kernels, zig-zag context
parallel attention, layer-range pipeline stages under the 1F1B schedule); DeepSeek-V4.1-family models
run with their routed experts split over the expert group (which spans the data x context ranks).
Gradients are averaged over the data group (and summed over tensor / context groups for replicated
parameters) and applied with fp32-master AdamW.  One JSON line per step goes to
``<run-dir>/metrics_rank0.jsonl``.

Plays the role of the reference's Megatron launches (``src/archlab/megatron/qwen38_flash_next_config.py:
140-260`` renders the parallel sizes; ``training/backends.py`` hands them to the trainer).
"""
from __future__ import annotations

import argparse
import faulthandler
import json
import os
import time
import zlib
from dataclasses import dataclass
from pathlib import Path

import torch
import torch.distributed as dist

from ..parallel import pp as ppar


@dataclass(frozen=True)
class Mesh:
    rank: int
    world: int
    tp: int
    cp: int
    dp: int
    pp: int

    @property
    def tp_i(self):
        return self.rank % self.tp

    @property
    def cp_i(self):
        return self.rank // self.tp % self.cp

    @property
    def dp_i(self):
        return self.rank // (self.tp * self.cp) % self.dp

    @property
    def pp_i(self):
        return self.rank // (self.tp * self.cp * self.dp)

    def rank_of(self, *, tp_i=None, cp_i=None, dp_i=None, pp_i=None) -> int:
        t = self.tp_i if tp_i is None else tp_i
        c = self.cp_i if cp_i is None else cp_i
        d = self.dp_i if dp_i is None else dp_i
        p = self.pp_i if pp_i is None else pp_i
        return ((p * self.dp + d) * self.cp + c) * self.tp + t

    def axis_ranks(self, axis: str) -> list[list[int]]:
        """Every group along ``axis`` (all ranks must create all groups, in this order)."""
        sizes = {"tp": self.tp, "cp": self.cp, "dp": self.dp, "pp": self.pp}
        others = [a for a in ("pp", "dp", "cp", "tp") if a != axis]
        groups = []

        def rec(fixed, rest):
            if not rest:
                groups.append([Mesh.rank_of(self, **{f"{axis}_i": i}, **{f"{k}_i": v for k, v in fixed.items()})
                               for i in range(sizes[axis])])
                return
            for v in range(sizes[rest[0]]):
                rec({**fixed, rest[0]: v}, rest[1:])

        rec({}, others)
        return groups

    def dpcp_ranks(self) -> list[list[int]]:
        """Groups over data x context (the expert-parallel / gradient-averaging span for experts)."""
        return [[self.rank_of(tp_i=t, pp_i=p, dp_i=d, cp_i=c) for d in range(self.dp) for c in range(self.cp)]
                for p in range(self.pp) for t in range(self.tp)]


def build_mesh(rank: int, world: int, tp: int, pp: int, cp: int) -> Mesh:
    mp = tp * pp * cp
    if world % mp:
        raise ValueError("world size must be divisible by tp x pp x cp")
    return Mesh(rank, world, tp, cp, world // mp, pp)


def make_groups(mesh: Mesh) -> dict:
    out = {}
    for axis in ("tp", "cp", "dp", "pp"):
        for ranks in mesh.axis_ranks(axis):
            g = dist.new_group(ranks) if len(ranks) > 1 else None
            if mesh.rank in ranks:
                out[axis] = g
    for ranks in mesh.dpcp_ranks():
        g = dist.new_group(ranks) if len(ranks) > 1 else None
        if mesh.rank in ranks:
            out["dpcp"] = g
    return out


def parse_args(argv=None):
    ap = argparse.ArgumentParser(description="tensor / pipeline / context / expert / data parallel training")
    ap.add_argument("--model", default="qwen35_tiny")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--cp", type=int, default=1)
    ap.add_argument("--ep", type=int, default=1)
    ap.add_argument("--sequence-parallel", action="store_true")
    ap.add_argument("--micro-batch", type=int, default=1)
    ap.add_argument("--global-batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp8_block", "fp8_tensor", "nvfp4"],
                    help="fp8_block: 1x128 / 128x128 power-of-two block scales, forward products on the block-scaled FP8 GEMM, "
                         "straight-through bf16 gradients; fp8_tensor: tensor-scaled e4m3 / e5m2 GEMMs; nvfp4: forward, "
                         "data- and weight-gradient products in NVFP4 (2-D weight blocks, stochastic rounding, Hadamard)")
    ap.add_argument("--model-set", action="append", default=[], metavar="KEY=VALUE",
                    help="factory models: override a field of the family's config (repeatable; values parse as JSON)")
    ap.add_argument("--native-linears", action="store_true",
                    help="run the bias-free nn.Linear layers of the model on the hand-written GEMM kernels")
    ap.add_argument("--fsdp", action="store_true",
                    help="factory models: shard the linear weights over the data group; the all-gather of a weight runs "
                         "inside the GEMM that consumes it")
    ap.add_argument("--fsdp-min-features", type=int, default=256, help="smallest linear side that is sharded")
    ap.add_argument("--fsdp-keep-gathered", action="store_true",
                    help="keep every gathered weight from the forward to the backward pass (no second gather)")
    ap.add_argument("--optimizer", default="adamw", choices=["adamw", "muon_split"],
                    help="muon_split: layer-wise distributed Muon with logical row splits on the parameters a model tags "
                         "for it (archlab_optimizer == 'muon'), sharded AdamW on the rest")
    ap.add_argument("--muon-lr", type=float, default=0.02)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--weight-decay", type=float, default=0.1)
    ap.add_argument("--grad-clip", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--run-dir", default="runs/mesh")
    ap.add_argument("--n-layer", type=int, default=0, help="override the preset's depth (0 keeps it)")
    ap.add_argument("--save-every", type=int, default=0, help="write a per-rank checkpoint every N steps (0: never)")
    ap.add_argument("--bounded-staging", action="store_true",
                    help="checkpoints: the local ranks of a host stage and write one at a time (bounds host memory)")
    ap.add_argument("--resume", action="store_true", help="continue from the newest checkpoint in --run-dir")
    ap.add_argument("--hang-dump-seconds", type=float, default=0.0,
                    help="a step that takes longer than this writes the Python stack of every thread of the rank to stderr "
                         "(re-armed every step; 0: off)")
    return ap.parse_args(argv)


# ------------------------------------------------------------------------------------------------
# models
# ------------------------------------------------------------------------------------------------
def _qwen35_config(name: str, a):
    from ..models.qwen35 import Qwen35Config

    kw = {"sequence_len": a.seq_len}
    if a.n_layer:
        kw["n_layer"] = a.n_layer
    if name == "qwen35_tiny":
        return Qwen35Config.tiny(**kw)
    if name == "qwen35_tiny_dense":
        return Qwen35Config.tiny(simplicial_every=0, **kw)
    if name == "qwen35_small":
        return Qwen35Config(**{**dict(vocab_size=32768, n_layer=4, hidden_size=1024, n_heads=8, n_kv_heads=4, intermediate_size=3072,
                                      simplicial_w1=16, simplicial_w2=64), **kw})
    if name == "qwen35_4b":
        return Qwen35Config(**kw)
    if name == "qwen35_4b_dense":
        return Qwen35Config(simplicial_every=0, **kw)
    raise ValueError(f"unknown model {name}")


class _Job:
    """Model + how one micro-batch runs on this rank.  ``stage(x, (ids, labels))`` follows the contract
    of ``parallel.pp.run_1f1b``."""

    def __init__(self, a, mesh: Mesh, groups: dict, device):
        self.mesh, self.groups, self.device, self.args = mesh, groups, device, a
        fam = a.model.split("_")[0]
        if a.model.startswith("factory:"):
            fam = "factory"
        if fam == "qwen35":
            from ..models.qwen35_tp import Qwen35TP

            cfg = _qwen35_config(a.model, a)
            tpg = None
            if mesh.tp > 1 and device.type == "cuda":
                from ..parallel.tp import TPGroup

                rows = a.seq_len // mesh.cp // mesh.tp
                # gathered operands and reduce-scattered outputs are always ``hidden_size`` wide
                tpg = TPGroup(rows, cfg.hidden_size, cfg.hidden_size, device, groups["tp"])
            stage_layers = ppar.split_layers(cfg.n_layer, mesh.pp)[mesh.pp_i]
            torch.manual_seed(a.seed)                         # same init stream on every rank of a stage
            self.model = Qwen35TP(cfg, tpg, world=mesh.tp, rank=mesh.tp_i, group=groups["tp"], layer_range=stage_layers,
                                  cp=(mesh.cp, mesh.cp_i, groups["cp"])).to(device)
            self._init_qwen(a.seed)
            self.act_shape = self.model.act_shape(a.seq_len)
            self.vocab = cfg.vocab_size
            self.kind = "tp"
        elif fam == "v41":
            from ..models.deepseek_v41 import V41Config, V41LM

            if mesh.tp > 1 or mesh.pp > 1 or mesh.cp > 1:
                raise ValueError("the V4.1 family runs under data + expert parallelism here")
            kw = {"sequence_len": a.seq_len, **({"n_layer": a.n_layer} if a.n_layer else {}),
                  **({"fp8": True} if a.precision == "fp8_block" else {})}
            presets = {"v41_tiny": V41Config.tiny, "v41_moe": V41Config,
                       "v41_small": lambda **k: V41Config(**{**dict(vocab_size=32768, n_layer=2, hidden_size=1024, n_heads=8,
                                                                    n_routed_experts=16, moe_inter=512, index_top_k=256), **k})}
            cfg = presets[a.model](**kw)
            ep_group = groups["dp"] if a.ep > 1 else None
            if a.ep > 1 and a.ep != mesh.dp:
                raise ValueError("expert parallel size must equal the data parallel size in this trainer")
            torch.manual_seed(a.seed)
            ep_buffers = None
            if ep_group is not None and device.type == "cuda":
                from ..parallel.ep import EPBuffers

                # worst case: every rank routes all of its slots to the experts of ONE rank (an untrained router can
                # come close); at 2 bytes x hidden per row the four buffers stay in the low GB range
                slots = a.micro_batch * a.seq_len * cfg.experts_top_k
                ep_buffers = EPBuffers(mesh.dp * slots, cfg.hidden_size, device, ep_group)
            self.ep_buffers = ep_buffers
            self.model = V41LM(cfg, ep_group, ep_buffers).to(device)
            self.model.init_weights()
            if ep_group is not None:                          # shared weights agree; every rank keeps its own experts
                for n, p in self.model.named_parameters():
                    if ".experts." not in n:
                        dist.broadcast(p.data, mesh.rank_of(dp_i=0), group=ep_group)
            self.act_shape, self.vocab, self.kind = None, cfg.vocab_size, "ep"
        elif a.model.startswith("factory:"):
            # any registered architecture family under data parallelism (model(ids, labels) -> loss)
            from ..models.factory import build_model

            if mesh.tp > 1 or mesh.pp > 1 or mesh.cp > 1 or a.ep > 1:
                raise ValueError("factory models run under data parallelism in this trainer")
            torch.manual_seed(a.seed)
            extra = {"sequence_len": a.seq_len, **({"n_layer": a.n_layer} if a.n_layer else {})}
            for item in getattr(a, "model_set", None) or []:            # KEY=VALUE overrides of the family's config
                key, _, val = item.partition("=")
                extra[key] = json.loads(val) if val and (val[0] in "[{\"-" or val[0].isdigit() or val in ("true", "false", "null")) else val
            self.model = build_model(a.model.split(":", 1)[1], extra, device=device)
            self.act_shape, self.kind = None, "dp"
            self.vocab = int(getattr(self.model.config, "vocab_size"))
        else:
            raise ValueError(f"unknown model family {fam}")
        if device.type == "cuda":
            self.model.to(torch.bfloat16)
        if a.precision == "fp8_tensor":
            from ..ops.fp8 import convert_linears

            self.fp8_layers = convert_linears(self.model)        # dense nn.Linear layers; expert and TP GEMMs stay bf16
        if a.precision == "nvfp4" or (a.precision == "fp8_block" and fam != "v41"):
            # block-scaled tensor-core products for the dense linears; what stays in BF16 and why is recorded
            from ..ops.blockscaled import convert_linears as to_block_scaled

            self.precision_report = to_block_scaled(self.model, "nvfp4" if a.precision == "nvfp4" else "fp8_block")
        if getattr(a, "native_linears", False) and not getattr(a, "fsdp", False):
            from ..ops.native_linear import convert_linears as to_native

            self.native_layers = to_native(self.model)           # nn.Linear layers onto the pair GEMM kernels
        self.fsdp = None
        if getattr(a, "fsdp", False):
            # fully-sharded linear weights over the data group: the gather runs inside the consuming GEMM kernel
            if self.kind != "dp" or mesh.dp < 2:
                raise ValueError("--fsdp shards the linears of a factory model over a data group of at least two ranks")
            from ..parallel.fsdp import FsdpGroup, shard_linears

            self.fsdp = FsdpGroup(device, groups["dp"], reshard_after_forward=not getattr(a, "fsdp_keep_gathered", False),
                                  grad_reduce="sum")      # the step scales every gradient by 1 / (accumulation x data ranks)
            shard_linears(self.model, self.fsdp, min_features=a.fsdp_min_features)

    def _init_qwen(self, seed: int) -> None:
        g = torch.Generator().manual_seed(seed)
        for name, p in self.model.named_parameters():
            if p.dim() < 2:
                continue
            # tensor-parallel shards of one matrix draw from different streams; replicated ones agree
            shard = self.mesh.tp_i if getattr(p, "tensor_model_parallel", False) else 0
            g.manual_seed(zlib.crc32(f"{seed}/{name}/{shard}".encode()))
            p.data.copy_(torch.randn(p.shape, generator=g).mul_(0.02).to(p.dtype))

    def expert_params(self) -> set:
        """Parameters that every data rank owns a different part of (updated locally, never reduced over the group):
        routed experts under expert parallelism, row shards of fully-sharded linears."""
        if self.fsdp is not None:
            return {layer.weight for layer in self.fsdp.layers}
        if self.kind != "ep" or not hasattr(self.model.layers[0].ffn, "local_experts"):
            return set()
        return {p for n, p in self.model.named_parameters() if ".experts." in n}

    def stage(self, x, mb):
        ids, labels = mb
        if self.kind == "tp":
            return self.model(ids, labels, x)
        return self.model(ids, labels)


class MasterAdamW:
    """AdamW on fp32 master copies; the model keeps its compute dtype."""

    def __init__(self, params, lr, weight_decay, betas=(0.9, 0.95), eps=1e-8):
        self.params = [p for p in params if p.requires_grad]
        self.master = [p.detach().float().clone() for p in self.params]
        self.m = [torch.zeros_like(w) for w in self.master]
        self.v = [torch.zeros_like(w) for w in self.master]
        self.lr, self.wd, self.betas, self.eps, self.t = lr, weight_decay, betas, eps, 0

    @torch.no_grad()
    def step(self, lr_scale: float = 1.0, grad_scale: float = 1.0):
        self.t += 1
        b1, b2 = self.betas
        grads = [(p.grad if p.grad is not None else torch.zeros_like(p)).float() * grad_scale for p in self.params]
        torch._foreach_mul_(self.m, b1)
        torch._foreach_add_(self.m, grads, alpha=1 - b1)
        torch._foreach_mul_(self.v, b2)
        torch._foreach_addcmul_(self.v, grads, grads, value=1 - b2)
        lr = self.lr * lr_scale
        c1, c2 = 1 - b1 ** self.t, 1 - b2 ** self.t
        decay = [w for w, p in zip(self.master, self.params) if p.dim() >= 2]
        if decay and self.wd:
            torch._foreach_mul_(decay, 1 - lr * self.wd)
        den = torch._foreach_sqrt(self.v)
        torch._foreach_div_(den, c2 ** 0.5)
        torch._foreach_add_(den, self.eps)
        torch._foreach_addcdiv_(self.master, self.m, den, value=-lr / c1)
        for p, w in zip(self.params, self.master):
            p.copy_(w)
            p.grad = None


# ------------------------------------------------------------------------------------------------
# run contract, checkpoints
# ------------------------------------------------------------------------------------------------
CONTRACT_KEYS = ("model", "tp", "pp", "cp", "ep", "micro_batch", "global_batch", "seq_len", "precision", "seed", "n_layer")


def run_contract(a, world: int) -> dict:
    """What must not change between the attempts of one run (a resume under a different contract is refused)."""
    from .precision_contract import FLAG_TO_PRECISION, precision_contract

    return {"format": "archlab-mesh-run-v1", "world_size": world, **{k: getattr(a, k) for k in CONTRACT_KEYS},
            "optimizer": getattr(a, "optimizer", "adamw"), "precision_contract": precision_contract(FLAG_TO_PRECISION[a.precision])}


def check_contract(run_dir: Path, contract: dict, resume: bool) -> int:
    """Writes RUN_CONTRACT.json on the first attempt, contracts/attempt-N.json on every attempt and
    LATEST_CONTRACT.json; returns the attempt number."""
    path = run_dir / "RUN_CONTRACT.json"
    (run_dir / "contracts").mkdir(parents=True, exist_ok=True)
    if path.exists():
        old = json.loads(path.read_text())
        if not resume:
            raise FileExistsError(f"{run_dir} already holds a run; pass --resume or choose a new directory")
        diff = sorted(k for k in set(old) | set(contract) if old.get(k) != contract.get(k))
        if diff:
            raise ValueError(f"resume contract differs in {diff}")
    else:
        if resume:
            raise FileNotFoundError("nothing to resume: no RUN_CONTRACT.json")
        path.write_text(json.dumps(contract, indent=2, sort_keys=True))
    attempt = len(list((run_dir / "contracts").glob("attempt-*.json"))) + 1
    (run_dir / "contracts" / f"attempt-{attempt}.json").write_text(json.dumps({**contract, "attempt": attempt, "time": time.time()},
                                                                              indent=2, sort_keys=True))
    (run_dir / "LATEST_CONTRACT.json").write_text(json.dumps({**contract, "attempt": attempt}, indent=2, sort_keys=True))
    return attempt


def staged_by_local_rank(write, *, local_rank: int, local_world: int, barrier) -> None:
    """Runs ``write()`` on one local rank of a host at a time.  Staging a rank's optimizer state for serialisation
    copies it to host memory; with large owner-sharded tables, all local ranks staging at once can exceed the host's
    memory, so the per-host order is bounded while every rank still writes its own file
    (src/archlab/megatron/checkpoint_staging.py:15-64)."""
    if local_world < 1 or not 0 <= local_rank < local_world:
        raise RuntimeError(f"invalid local checkpoint topology: rank={local_rank}, world={local_world}")
    import gc

    for turn in range(local_world):
        if turn == local_rank:
            write()
            gc.collect()                      # hand the staged host copies back before the next rank takes its turn
        barrier()


def save_checkpoint(run_dir: Path, step: int, rank: int, job, opt, *, bounded_staging: bool = False) -> None:
    """Every rank writes its own model shard and optimizer slice; rank 0 writes the step marker LAST."""
    d = run_dir / "checkpoints" / f"step_{step:07d}"
    d.mkdir(parents=True, exist_ok=True)

    def write():
        state = {"step": step, "model": job.model.state_dict(), "zero": opt.zero.state_dict(),
                 "experts": None if opt.experts is None else {"t": opt.experts.t, "master": opt.experts.master, "m": opt.experts.m,
                                                              "v": opt.experts.v},
                 "muon": None if getattr(opt, "muon", None) is None else opt.muon.state_dict(),
                 "rng": torch.get_rng_state()}
        tmp = d / f".rank{rank:03d}.pt.tmp"
        torch.save(state, tmp)
        os.replace(tmp, d / f"rank{rank:03d}.pt")

    if bounded_staging and dist.is_initialized():
        staged_by_local_rank(write, local_rank=int(os.environ.get("LOCAL_RANK", rank)),
                             local_world=int(os.environ.get("LOCAL_WORLD_SIZE", dist.get_world_size())), barrier=dist.barrier)
    else:
        write()
    if dist.is_initialized():
        dist.barrier()
    if rank == 0:
        (run_dir / "checkpoints" / "latest_checkpointed_iteration.txt").write_text(f"{step}\n")


def load_checkpoint(run_dir: Path, rank: int, job, opt) -> int:
    marker = run_dir / "checkpoints" / "latest_checkpointed_iteration.txt"
    if not marker.exists():
        return 0
    step = int(marker.read_text().strip())
    state = torch.load(run_dir / "checkpoints" / f"step_{step:07d}" / f"rank{rank:03d}.pt", map_location="cpu", weights_only=False)
    opt.zero.load_state_dict(state["zero"])
    with torch.no_grad():                                    # parameters are views of the flat buffer: copy in place
        for name, p in job.model.named_parameters():
            p.copy_(state["model"][name])
        for name, b in job.model.named_buffers():
            if name in state["model"]:
                b.copy_(state["model"][name])
    if getattr(opt, "muon", None) is not None and state.get("muon") is not None:
        opt.muon.load_state_dict(state["muon"])
    if opt.experts is not None and state["experts"] is not None:
        e = state["experts"]
        opt.experts.t = e["t"]
        for dst, src in zip(opt.experts.master + opt.experts.m + opt.experts.v, e["master"] + e["m"] + e["v"]):
            dst.copy_(src)
    torch.set_rng_state(state["rng"])
    return step


# ------------------------------------------------------------------------------------------------
# step
# ------------------------------------------------------------------------------------------------
def _allreduce(t, group, op=dist.ReduceOp.SUM):
    if group is not None:
        dist.all_reduce(t, op=op, group=group)


class MeshOptimizer:
    """ZeRO-sharded AdamW over the data group for everything that is averaged over it, plus a local
    AdamW for routed experts (each data rank owns different experts)."""

    def __init__(self, job: _Job, lr: float, weight_decay: float):
        from ..optim.zero import ZeroAdamW

        self.job = job
        experts = job.expert_params()
        shared = [p for p in job.model.parameters() if p not in experts and p.requires_grad]
        self.muon = None
        if getattr(job.args, "optimizer", "adamw") == "muon_split":
            from ..optim.split_muon import SplitRowsMuon

            if job.kind != "dp":
                raise ValueError("--optimizer muon_split runs on data-parallel (factory) models")
            # sums over the data group like the sharded AdamW: the step applies 1 / (accumulation x data ranks) to both
            self.muon = SplitRowsMuon(job.model.named_parameters(), lr=job.args.muon_lr, weight_decay=weight_decay,
                                      group=job.groups["dp"], average=False)
            taken = {id(p) for p in self.muon.params}
            shared = [p for p in shared if id(p) not in taken]
        is_repl = lambda p: not getattr(p, "tensor_model_parallel", False)
        shared.sort(key=lambda p: (p.dim() < 2, not is_repl(p)))      # decayed replicated | decayed sharded | plain
        self.zero = ZeroAdamW(shared, lr=lr, weight_decay=weight_decay, group=job.groups["dp"])
        self.experts = MasterAdamW(list(experts), lr, weight_decay) if experts else None
        repl = [p for p in shared if is_repl(p)]
        dec = [p for p in repl if p.dim() >= 2]
        plain = [p for p in repl if p.dim() < 2]
        self.repl_ranges = [self.zero.range_of(g) for g in (dec, plain) if g]
        self.zero.zero_grad()

    def reduce_and_norm(self, scale: float) -> float:
        job, g, z = self.job, self.job.groups, self.zero
        if job.kind == "tp":
            for a, b in self.repl_ranges:                              # every tensor rank saw different rows
                _allreduce(z.flat_g[a:b], g["tp"])
            _allreduce(z.flat_g, g["cp"])
        z.reduce_gradients()
        sq_all, sq_repl = z.grad_sq_norm(), z.grad_sq_norm(self.repl_ranges)
        both = torch.stack([sq_all, sq_repl])
        _allreduce(both, g["dp"])
        if self.muon is not None:                                       # identical on every rank after its reduction
            self.muon.reduce_gradients()
            both[0] = both[0] + self.muon.grad_sq_norm()
        sharded = both[0] - both[1]
        if self.experts is not None:
            e = torch.stack([p.grad.float().pow(2).sum() for p in self.experts.params if p.grad is not None]).sum()
            _allreduce(e, g["dp"])
            sharded = sharded + e
        if job.kind == "tp":
            _allreduce(sharded, g["tp"])
        total = sharded + both[1]
        _allreduce(total, g["pp"])
        return float(total.sqrt()) * scale

    def step(self, lr_scale: float, grad_scale: float) -> None:
        fsdp = getattr(self.job, "fsdp", None)
        if fsdp is not None:
            fsdp.sync()                                   # no peer still reads the shards this step rewrites
        self.zero.step(lr_scale=lr_scale, grad_scale=grad_scale)
        if self.muon is not None:
            self.muon.step(lr_scale=lr_scale, grad_scale=grad_scale)
        if self.experts is not None:
            self.experts.step(lr_scale=lr_scale, grad_scale=grad_scale)
        if fsdp is not None:
            fsdp.sync()                                   # the new shards are visible before the next forward


def train(a, *, on_step=None) -> list[float]:
    rank, world, device = _init_distributed()
    mesh = build_mesh(rank, world, a.tp, a.pp, a.cp)
    if a.global_batch % (a.micro_batch * mesh.dp):
        raise SystemExit("global batch must be a multiple of micro batch x data parallel size")
    if a.micro_batch != 1 and a.model.startswith("qwen35"):
        raise SystemExit("sequence-parallel models take one sequence per micro-batch")
    accum = a.global_batch // (a.micro_batch * mesh.dp)
    groups = make_groups(mesh) if world > 1 else {k: None for k in ("tp", "cp", "dp", "pp", "dpcp")}
    job = _Job(a, mesh, groups, device)
    opt = MeshOptimizer(job, a.lr, a.weight_decay)
    links = ppar.StageLinks(mesh.pp_i, mesh.pp, mesh.rank_of(pp_i=mesh.pp_i - 1) if mesh.pp_i else None,
                            mesh.rank_of(pp_i=mesh.pp_i + 1) if mesh.pp_i + 1 < mesh.pp else None)
    run_dir = Path(os.environ.get(a.run_dir[4:], "runs/mesh") if a.run_dir.startswith("env:") else a.run_dir)
    log, receipts = None, None
    refusal = None
    if rank == 0:
        from ..ckpt.formats import RunReceipts

        try:
            run_dir.mkdir(parents=True, exist_ok=True)
            attempt = check_contract(run_dir, run_contract(a, world), a.resume)
            (run_dir / "config.json").write_text(json.dumps({"args": vars(a), "world_size": world, "data_parallel": mesh.dp,
                                                             "grad_accum_steps": accum, "attempt": attempt}, indent=2))
            (run_dir / "PARALLELISM.json").write_text(json.dumps({"tensor": mesh.tp, "pipeline": mesh.pp, "context": mesh.cp,
                                                                  "expert": a.ep, "data": mesh.dp, "world_size": world,
                                                                  "order": "tensor fastest, then context, data, pipeline"}, indent=2))
            (run_dir / "MODEL_SHAPES.json").write_text(json.dumps({n: list(p.shape) for n, p in job.model.named_parameters()}, indent=1))
            receipts = RunReceipts(run_dir, {"args": vars(a), "world_size": world})
            if a.resume:                                         # the stop that ended the previous attempt is consumed
                (run_dir / "STOP_REQUESTED.json").unlink(missing_ok=True)
                (run_dir / "STOPPED.json").unlink(missing_ok=True)
            log = open(run_dir / "metrics_rank0.jsonl", "a")
        except Exception as exc:                                 # told to the other ranks below, then raised here
            refusal = exc
    if world > 1:
        # rank 0's verdict on the run directory reaches every rank: a refused contract or a closed
        # directory ends all of them here instead of leaving the others in a collective until it times out
        verdict = [None if refusal is None else f"{type(refusal).__name__}: {refusal}"]
        dist.broadcast_object_list(verdict, src=0)
        if rank != 0 and verdict[0] is not None:
            dist.destroy_process_group()
            raise RuntimeError(f"rank 0 refused the run directory: {verdict[0]}")
    if refusal is not None:
        if world > 1:
            dist.destroy_process_group()
        raise refusal
    start = load_checkpoint(run_dir, rank, job, opt) if a.resume else 0
    from . import health

    if world > 1:
        health.collective_probe(device, timeout_seconds=300.0)   # an absent rank fails here, not in the first step
    guard = health.FiniteGuard(device)
    stop = health.StopConsensus(run_dir, device)
    beat = health.Heartbeat(run_dir, rank=rank)
    from ..data.synthetic import ZipfTokens

    # every rank of a (tensor, context, pipeline) slice reads the data of its data-parallel index
    gen = ZipfTokens(job.vocab, a.seq_len, a.micro_batch * accum, seed=a.seed, rank=mesh.dp_i, pin=False)
    act_dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    losses = []
    scale = 1.0 / (accum * mesh.dp)
    cuda = device.type == "cuda"
    reached, stopped_early = start, False
    watchdog = float(getattr(a, "hang_dump_seconds", 0.0) or 0.0)
    for step in range(start, a.steps):
        t0 = time.perf_counter()
        if watchdog > 0:                                         # where is every thread if this step does not come back
            faulthandler.dump_traceback_later(watchdog, repeat=True, exit=False)
        if cuda:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        block = gen.block(step).to(device).long()              # [micro*accum, T+1]
        mbs = [(block[i * a.micro_batch:(i + 1) * a.micro_batch, :-1], block[i * a.micro_batch:(i + 1) * a.micro_batch, 1:])
               for i in range(accum)]
        if mesh.pp > 1:
            loss = ppar.run_1f1b(links, job.stage, mbs, act_shape=job.act_shape, act_dtype=act_dtype, device=device)
        else:
            loss = torch.zeros((), device=device)
            for mb in mbs:
                l = job.stage(None, mb)
                l.backward()
                loss = loss + l.detach()
        gnorm = opt.reduce_and_norm(scale)
        clip = min(1.0, a.grad_clip / (gnorm + 1e-6)) if a.grad_clip > 0 else 1.0
        warm = min(1.0, (step + 1) / max(1, min(10, a.steps // 10)))
        opt.step(warm, scale * clip)
        # mean loss of the step: partial sums live on the last stage's tensor/context ranks
        loss = loss.float() * scale
        if job.kind == "tp":
            _allreduce(loss, groups["tp"])
            _allreduce(loss, groups["cp"])
        _allreduce(loss, groups["dp"])
        _allreduce(loss, groups["pp"])
        if cuda:                                                 # device time of the step, max over ranks
            ev1.record()
            torch.cuda.synchronize()
            ms = torch.tensor([ev0.elapsed_time(ev1)], device=device)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            dt = float(ms) / 1e3
        else:
            dt = time.perf_counter() - t0
        losses.append(float(loss))
        if cuda:
            from ..ops import native

            if native.available():
                native.check_status()                            # an expired device-side wait (peer barrier, flag) ends the run here
        dropped = None
        if getattr(job, "ep_buffers", None) is not None and getattr(job.model.config, "expert_capacity_factor", None) is not None:
            dropped = job.ep_buffers.check_overflow()["dropped_rows"]      # rows past the expert row bound (tokens dropped)
        guard.check(step + 1, losses[-1], gnorm)
        beat.beat(step=step + 1, loss=losses[-1])
        if log is not None:
            log.write(json.dumps({"step": step + 1, "loss": losses[-1], "grad_norm": gnorm, "step_seconds": dt, "dropped_expert_rows": dropped,
                                  "tokens_per_second": a.global_batch * a.seq_len / dt,
                                  "timing": "cuda events, max over ranks" if cuda else "host clock",
                                  "peak_mem_gib": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2) if cuda else 0.0,
                                  "parallelism": f"tp{mesh.tp} pp{mesh.pp} cp{mesh.cp} ep{a.ep} dp{mesh.dp}"}) + "\n")
            log.flush()
        if on_step is not None:
            on_step(step, losses[-1])
        stopping = stop.should_stop()
        if (a.save_every and ((step + 1) % a.save_every == 0 or step + 1 == a.steps)) or stopping:
            save_checkpoint(run_dir, step + 1, rank, job, opt, bounded_staging=getattr(a, "bounded_staging", False))
        reached = step + 1
        if stopping:                                             # every rank leaves at the same step, after the checkpoint
            stop.acknowledge(step + 1, rank)
            stopped_early = reached < a.steps
            break
    if watchdog > 0:
        faulthandler.cancel_dump_traceback_later()
    if receipts is not None:
        outcome = {"final_loss": losses[-1] if losses else None, "steps": reached, "step_budget": a.steps}
        if stopped_early:
            # a graceful stop leaves STOPPED.json + the checkpoint and no completion marker, so that
            # --resume can continue it (src/archlab/megatron/simplicial_pilot.py:457-460)
            receipts.stopped(outcome)
        else:
            receipts.finish(outcome)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return losses


def _init_distributed():
    if "RANK" not in os.environ:
        return 0, 1, torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    rank, local = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", 0))
    if torch.cuda.is_available():
        torch.cuda.set_device(local)
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return rank, dist.get_world_size(), torch.device("cuda", local)
    if not dist.is_initialized():
        dist.init_process_group("gloo")
    return rank, dist.get_world_size(), torch.device("cpu")


def main(argv=None) -> int:
    train(parse_args(argv))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
