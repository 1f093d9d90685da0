"""Headline benchmark: training throughput of the nanochat-style speedrun GPT d20.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched under torchrun)
    python bench.py --impl reference ...                      (the reference arm)
    python bench.py --impl eager ...                          (this repo's cuBLAS/SDPA/NCCL decomposition)
    python bench.py --config qwen35_4b_simplicial | v41_moe   (the mesh trainer's step on the larger configurations)

Config (BASELINE.json, config 2): 20 layers, d_model 1280, 10 heads x 128, QK-norm, vocab 65536,
seq 2048, bf16, Muon + AdamW, ZeRO-1 style gradient sync inside the optimizer.  Weak scaling:
32 sequences (64 Ki tokens) per GPU per step, i.e. 512 Ki tokens per step on 8 GPUs.  Tokens are
Zipf(1.1) ids from seed 0 and weights are random-init, since no dataset or checkpoint is reachable.

Rank 0 prints ONE JSON line.  ``value`` is device-timed (CUDA events around K steps whose inputs are
already on the device, max over ranks); ``e2e`` times K further steps through the public
``Trainer.train_step`` call, which copies each step's tokens from pinned host memory and reads the
loss back.  The step's working set (tens of GB of activations and weights) is far larger than the
126 MB L2, so no explicit L2 flush is needed between iterations.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int, period: float = 0.2):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = None
        self._halt = threading.Event()

    def run(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = int(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            names = {
                "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
            }
            get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                nv.nvmlDeviceGetCurrentClocksThrottleReasons
            while not self._halt.is_set():
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                mask = int(get_reasons(h))
                for k, bit in names.items():
                    if mask & bit:
                        self.reasons.add(k)
                time.sleep(self.period)
        except Exception as exc:  # pragma: no cover - NVML missing
            self.reasons.add(f"nvml_unavailable:{type(exc).__name__}")

    def stop(self) -> dict:
        self._halt.set()
        self.join(timeout=2.0)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "eager"])
    ap.add_argument("--local-batch", type=int, default=32, help="sequences per GPU per step")
    ap.add_argument("--micro-batch", type=int, default=None,
                    help="sequences per forward/backward (default: 16 here, 32 = the stock "
                         "--device-batch-size in the reference arm)")
    ap.add_argument("--depth", type=int, default=20)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--vocab", type=int, default=65536)
    ap.add_argument("--window-pattern", default="SSSL", help="the speedrun script's default in both arms")
    ap.add_argument("--no-compile", action="store_true", help="reference arm: skip torch.compile")
    # optimizer settings shared by both arms (the reference script's defaults, base_train.py:499-522)
    ap.add_argument("--matrix-lr", type=float, default=0.02)
    ap.add_argument("--embedding-lr", type=float, default=0.3)
    ap.add_argument("--unembedding-lr", type=float, default=0.008)
    ap.add_argument("--scalar-lr", type=float, default=0.5)
    ap.add_argument("--weight-decay", type=float, default=0.28)
    ap.add_argument("--config", default="d20", choices=["d20", "qwen35_4b_simplicial", "v41_moe"],
                    help="d20: the speedrun GPT (headline); the others time the mesh trainer's step")
    ap.add_argument("--precision", default="bf16", choices=["bf16", "fp8_block", "nvfp4"],
                    help="configurations 3 and 4 only: compute precision of the linear layers (the d20 headline is bf16)")
    ap.add_argument("--per-gpu-batch", type=int, default=0, help="configurations 3 and 4: sequences per GPU per step (0: 16 / 4)")
    ap.add_argument("--kernel-times", action="store_true",
                    help="after the timed runs: two more steps under the torch profiler's CUDA activity records, kernel "
                         "durations summed by kernel to stderr (in-situ shares at the power-capped clock; never a bench value)")
    ap.add_argument("--no-extra", action="store_true", help="skip the kernel metrics appended to the d20 line")
    args = ap.parse_args()
    if args.warmup < 3:
        raise SystemExit("at least 3 warm-up steps are required")

    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import reference_arm

        if args.micro_batch is None:
            args.micro_batch = min(32, args.local_batch)
        why = reference_arm.ensure_reference_tree()
        if why is not None:
            print(json.dumps({"impl": "reference", "unavailable": why}))
            return
        out = reference_arm.run(args, ClockSampler)
        if out is not None:
            print(json.dumps(out))
        return
    if args.config != "d20":
        return mesh_config(args)
    if args.micro_batch is None:
        args.micro_batch = min(16, args.local_batch)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from archlab_b200.data.synthetic import ZipfTokens
    from archlab_b200.models.nanochat import GPTConfig
    from archlab_b200.ops import native
    from archlab_b200.train.speedrun import Trainer, TrainerConfig

    mcfg = GPTConfig.from_depth(args.depth, sequence_len=args.seq_len, vocab_size=args.vocab,
                                compute_dtype=torch.bfloat16, matrix_init_recipe="normal-0.02",
                                window_pattern=args.window_pattern)
    tcfg = TrainerConfig(model=mcfg, micro_batch=args.micro_batch, num_iterations=10000,
                         matrix_lr=args.matrix_lr, embedding_lr=args.embedding_lr,
                         unembedding_lr=args.unembedding_lr, scalar_lr=args.scalar_lr,
                         weight_decay=args.weight_decay,
                         # eager arm: module forward / autograd (cuBLAS + SDPA) and the NCCL optimizer from the start
                         use_engine=args.impl != "eager", zero_impl="nccl" if args.impl == "eager" else "auto")
    trainer = Trainer(tcfg, device=dev)
    data = ZipfTokens(args.vocab, args.seq_len, args.local_batch, s=1.1, seed=0, rank=rank, pin=True)
    n_blocks = args.warmup + 2 * args.steps
    host_blocks = [data.block(i) for i in range(n_blocks)]
    dev_blocks = [b.to(dev) for b in host_blocks[: args.warmup + args.steps]]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (untimed)
    for i in range(args.warmup):
        trainer.train_step_device(dev_blocks[i])
    barrier()
    if trainer.engine is not None:
        native.check_status()

    # ---- device-timed region
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = native.launch_count() if native.available() else 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        loss = trainer.train_step_device(dev_blocks[args.warmup + i])
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)
    launches = (native.launch_count() - launches0) if native.available() else 0
    last_loss = float(loss.item())

    # ---- end-to-end region: public API, pinned host inputs, loss read back every step
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        last_loss = trainer.train_step(host_blocks[args.warmup + args.steps + i])
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3
    barrier()
    clocks = sampler.stop()
    if trainer.engine is not None:
        native.check_status()
    if args.kernel_times and rank == 0:
        kernel_times(trainer, host_blocks)

    times = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(times[0]), float(times[1])
    tokens_per_step = args.local_batch * args.seq_len * world
    value = tokens_per_step * args.steps / (dev_ms / 1e3)
    e2e_value = tokens_per_step * args.steps / (e2e_ms / 1e3)
    h2d = host_blocks[0].numel() * host_blocks[0].element_size()
    if rank == 0:
        out = {
            "metric": "train tokens/sec/box", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic: Zipf(1.1) token ids from seed 0, random-init weights",
            "impl": args.impl,
            "config": {
                "model": f"nanochat-speedrun-d{args.depth} ({mcfg.n_layer}L, d_model {mcfg.n_embd}, "
                         f"{mcfg.n_head}x{mcfg.head_dim} heads, vocab {args.vocab})",
                "global_batch": tokens_per_step, "seq_len": args.seq_len,
                "parallelism": f"dp{world} (ZeRO-1 Muon/AdamW inside the optimizer)",
                "micro_batch_sequences": args.micro_batch, "window_pattern": args.window_pattern,
                "l2": "working set per step far exceeds the 126 MB L2; no explicit flush",
            },
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": int(launches),
            "final_loss": last_loss,
        }
        if args.impl == "native" and not args.no_extra:
            from archlab_b200.bench_kernels import simplicial_headline

            del trainer
            torch.cuda.empty_cache()
            out["extra_metrics"] = simplicial_headline()
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


def kernel_times(trainer, host_blocks, steps: int = 2) -> None:
    """Kernel durations of ``steps`` training steps, summed by kernel name, largest first, to stderr."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for i in range(steps):
            trainer.train_step(host_blocks[i % len(host_blocks)])
        torch.cuda.synchronize()
    groups: dict[str, list] = {}
    for e in prof.key_averages():
        name = e.key.split("(")[0].split("<")[0].strip()[-64:]
        g = groups.setdefault(name, [0.0, 0])
        g[0] += e.self_device_time_total / 1e3 / steps
        g[1] += e.count // steps
    total = sum(ms for ms, _ in groups.values())
    print(f"kernel time per step {total:.1f} ms", file=sys.stderr)
    for name, (ms, n) in sorted(groups.items(), key=lambda kv: -kv[1][0])[:30]:
        print(f"{ms:9.2f} ms {n:5d}x  {name}", file=sys.stderr)


def mesh_config(args) -> None:
    """Configurations 3 and 4 through the mesh trainer (``archlab_b200.train.mesh_train.train``, the call a user
    makes): per-GPU work is fixed (16 resp. 4 sequences per GPU per step), every step copies its token block from the
    host and reads the loss back.  ``value`` sums the trainer's own per-step device times (CUDA events, max over
    ranks); ``e2e`` is the wall clock around the same steps."""
    import tempfile

    import torch

    from archlab_b200.ops import native
    from archlab_b200.train import mesh_train

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    total = args.warmup + args.steps
    run_dir = tempfile.mkdtemp(prefix="bench-mesh-") if rank == 0 else ""
    if args.config == "qwen35_4b_simplicial":
        tp = 2 if world >= 2 else 1
        seq, per_gpu = 8192, args.per_gpu_batch or 16
        argv = ["--model=qwen35_4b", f"--tp={tp}", "--seq-len=8192", f"--global-batch={per_gpu * world}"]
        if tp > 1:
            argv.append("--sequence-parallel")
        par = f"tp{tp}+sp x zero-dp{world // tp}"
        model = "Qwen3.5-4B-like dense (36L, hidden 2560, 32/8 heads x 128, FFN 9728, vocab 151936), every 4th layer 2-simplicial 32x512"
    else:
        if world < 4:
            raise SystemExit("v41_moe keeps 64 experts' weights, gradients and optimizer state on the expert-parallel group: "
                             "it needs at least 4 GPUs of 180 GB")
        seq, per_gpu = 4096, args.per_gpu_batch or 4
        argv = ["--model=v41_moe", f"--ep={world}", "--seq-len=4096", "--micro-batch=1", f"--global-batch={per_gpu * world}"]
        par = f"ep{world} (= dp{world})"
        model = "DeepSeek-V4.1-style MoE (24L, hidden 2048, 64 routed experts FFN 1408 top-6 + 2 shared, DSA top-2048, 4 HC streams)"
    argv += [f"--precision={args.precision}", "--hang-dump-seconds=120", f"--steps={total}", f"--run-dir={run_dir or tempfile.gettempdir() + '/bench-mesh-other'}"]
    marks = {}
    sampler = ClockSampler(int(os.environ.get("LOCAL_RANK", "0")))

    def on_step(step, loss):
        if step + 1 == args.warmup:
            torch.cuda.synchronize()
            sampler.start()
            marks["t0"], marks["l0"] = time.perf_counter(), native.launch_count()
        if step + 1 == total:
            torch.cuda.synchronize()
            marks["t1"], marks["l1"], marks["loss"] = time.perf_counter(), native.launch_count(), loss

    mesh_train.train(mesh_train.parse_args(argv), on_step=on_step)
    clocks = sampler.stop()
    if rank != 0:
        return
    rows = [json.loads(line) for line in open(os.path.join(run_dir, "metrics_rank0.jsonl"))]
    dev_s = sum(r["step_seconds"] for r in rows[args.warmup:total])
    tokens = per_gpu * world * seq
    e2e_s = marks["t1"] - marks["t0"]
    print(json.dumps({
        "metric": "train tokens/sec/box", "value": tokens * args.steps / dev_s, "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_s / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": args.precision,
        "data": "synthetic: Zipf(1.1) token ids from seed 0, random-init weights", "impl": "native",
        "config": {"model": model, "global_batch": tokens, "seq_len": seq, "parallelism": par,
                   "l2": "working set per step far exceeds the 126 MB L2; no explicit flush"},
        "clocks": clocks,
        "e2e": {"value": tokens * args.steps / e2e_s, "unit": "tokens/s", "h2d_bytes_per_step": per_gpu * (seq + 1) * 8,
                "d2h_bytes_per_step": 4, "ms_per_step": e2e_s / args.steps * 1e3},
        "gpu_launches": int(marks["l1"] - marks["l0"]), "final_loss": marks["loss"],
        "peak_mem_gib": rows[-1].get("peak_mem_gib")}))


if __name__ == "__main__":
    main()
