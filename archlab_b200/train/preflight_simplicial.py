"""Kernel preflight for 2-simplicial attention: a runnable gate that writes a receipt.

    python -m archlab_b200.train.preflight_simplicial --output receipt.json [--correctness-only] [--sequence N]

What it establishes before any training launch (the reference's gate does the same for its Triton kernels,
src/archlab/qualification/simplicial_attention.py:30-231):

1. a numerical ladder: outputs and all five input gradients of the dispatching op (the sm_100a kernels for bf16,
   head_dim 128 on a GPU; the PyTorch statement otherwise) against an FP64 evaluation of the definition, for a list
   of (length, short window, long window) cases that includes single-token, window-1 and ragged-edge shapes;
2. causality: adding a large perturbation to the second half of any key / value input leaves the first half of the
   output bit-identical;
3. (GPU only) forward and forward+backward latency of the attention core for a global causal arm, a local-window
   arm (both through the framework's flash kernel) and the simplicial arm at three window pairs, with peak memory.

The process caps itself at a quarter of the device memory so that a preflight next to a serving process cannot
crowd it out.  The receipt is rewritten atomically after every case, so a failed or interrupted run still leaves the
evidence gathered so far; ``status`` ends as ``passed`` or ``failed`` and the exit code follows it.
"""
from __future__ import annotations

import argparse
import hashlib
import json
import platform
import socket
import sys
import time
from pathlib import Path

import torch

from ..contracts.substrate import atomic_write_json
from ..ops.simplicial import simplicial_attention, simplicial_attention_reference

LADDER = ((1, 1, 1), (17, 1, 1), (17, 3, 8), (35, 16, 32), (65, 8, 128), (529, 32, 512))
INPUT_NAMES = ("q", "k1", "k2", "v1", "v2")
WINDOW_PAIRS = ((8, 64), (16, 128), (32, 512))


def _make_inputs(batch, n, heads, kv_heads, dim, dtype, device, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    shapes = [(batch, n, heads, dim)] + [(batch, n, kv_heads, dim)] * 4
    return [(torch.randn(s, generator=g) * 0.7).to(device=device, dtype=dtype).requires_grad_(True) for s in shapes]


def correctness_case(n: int, w1: int, w2: int, dtype, *, device, batch: int = 1, heads: int = 4, kv_heads: int = 2,
                     dim: int = 128, positions=None) -> dict:
    inputs = _make_inputs(batch, n, heads, kv_heads, dim, dtype, device, seed=1000 + n)
    out = simplicial_attention(*inputs, w1, w2)
    upstream = torch.randn(out.shape, generator=torch.Generator().manual_seed(7)).to(out)
    out.backward(upstream)
    oracle_in = [x.detach().double().cpu().requires_grad_(True) for x in inputs]
    oracle = simplicial_attention_reference(*oracle_in, w1, w2)
    oracle.backward(upstream.double().cpu())
    rows = slice(None) if positions is None else torch.tensor([p for p in positions if p < n])

    def err(got, want):
        got, want = got.detach().double().cpu()[:, rows], want.detach()[:, rows]
        return {"relative_l2": float((got - want).norm() / want.norm().clamp_min(1e-30)), "max_absolute": float((got - want).abs().max())}

    errors = {"output": err(out, oracle)}
    errors.update({f"d{name}": err(x.grad, y.grad) for name, x, y in zip(INPUT_NAMES, inputs, oracle_in)})
    limit = 0.025 if dtype == torch.bfloat16 else 1e-4
    numerics = all(e["relative_l2"] <= limit or e["max_absolute"] <= limit * 0.01 for e in errors.values())
    finite = all(bool(torch.isfinite(x.grad).all()) for x in inputs)
    half = max(1, n // 2)
    causal = True
    for moved in (1, 2, 3, 4):                                    # every key / value input, one at a time
        altered = [x.detach().clone() for x in inputs]
        altered[moved][:, half:] += 10
        again = simplicial_attention(*altered, w1, w2)
        causal = causal and torch.equal(again[:, :half], out.detach()[:, :half])
    return {"batch": batch, "sequence": n, "heads": [heads, kv_heads], "head_dim": dim, "windows": [w1, w2], "dtype": str(dtype),
            "oracle_dtype": "float64", "query_positions": positions, "errors": errors, "relative_l2_limit": limit,
            "gradients_finite": finite, "future_perturbation_exact": causal, "passed": numerics and finite and causal}


def benchmark_case(kind: str, window, *, sequence: int, batch: int, repetitions: int) -> dict:
    """Attention core only (no projections, norms, optimizer): 16 query / 4 KV heads of 128, bf16."""
    from ..ops.attention import causal_attention

    q, k1, k2, v1, v2 = inputs = _make_inputs(batch, sequence, 16, 4, 128, torch.bfloat16, "cuda", seed=42)
    upstream = torch.randn_like(q)

    def forward():
        if kind == "simplicial":
            return simplicial_attention(*inputs, *window)
        return causal_attention(q, k1, v1, window=-1 if kind == "global" else window[1] - 1)

    def step():
        for x in inputs:
            x.grad = None
        forward().backward(upstream)

    for _ in range(3):
        with torch.no_grad():
            forward()
        step()
    torch.cuda.synchronize()
    torch.cuda.reset_peak_memory_stats()
    fwd, both = [], []
    for _ in range(repetitions):
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record()
        with torch.no_grad():
            forward()
        e1.record()
        step()
        e2.record()
        e2.synchronize()
        fwd.append(e0.elapsed_time(e1))
        both.append(e1.elapsed_time(e2))
    return {"kind": kind, "implementation": "sm_100a tcgen05 kernels of this package", "windows": list(window), "batch": batch,
            "sequence": sequence, "query_heads": 16, "kv_heads": 4, "head_dim": 128, "forward_ms": fwd, "forward_backward_ms": both,
            "peak_allocated_bytes": torch.cuda.max_memory_allocated(),
            "scope": "attention core only; no projections, optimizer, or model training"}


def run(output: Path, *, sequence: int = 2048, batch: int = 1, repetitions: int = 20, correctness_only: bool = False,
        device: str | None = None, ladder=LADDER) -> dict:
    if output.exists():
        raise ValueError(f"refusing to overwrite {output}")
    if min(sequence, batch, repetitions) < 1:
        raise ValueError("benchmark dimensions and repetitions must be positive")
    device = device or ("cuda" if torch.cuda.is_available() else "cpu")
    on_gpu = device.startswith("cuda")
    if on_gpu:
        torch.cuda.set_device(0)
        torch.cuda.set_per_process_memory_fraction(0.25)           # a preflight must not crowd out a co-resident service
    here = Path(__file__).resolve().parent.parent
    sources = [here / "ops/simplicial.py", here / "ops/simplicial_cuda.py", here / "csrc/simplicial_fwd.cu", here / "csrc/simplicial_bwd.cu"]
    evidence = {"status": "running", "host": socket.gethostname(), "python": sys.executable, "python_version": platform.python_version(),
                "torch_version": torch.__version__, "cuda_version": torch.version.cuda, "device": device,
                "gpu": str(torch.cuda.get_device_properties(0)) if on_gpu else None,
                "source_sha256": {str(p.relative_to(here)): hashlib.sha256(p.read_bytes()).hexdigest() for p in sources if p.exists()},
                "started_unix": time.time(), "training_started": False, "correctness": [], "benchmarks": []}
    save = lambda: atomic_write_json(output, evidence)
    output.parent.mkdir(parents=True, exist_ok=True)
    save()
    try:
        dtypes = (torch.float32, torch.bfloat16) if on_gpu else (torch.float32,)
        for dtype in dtypes:
            for n, w1, w2 in ladder:
                positions = [0, 31, 511, 512, 528] if n == 529 else None
                case = correctness_case(n, w1, w2, dtype, device=device, batch=2 if n == 17 else 1, positions=positions)
                evidence["correctness"].append(case)
                save()
                print(json.dumps(case), flush=True)
                if not case["passed"]:
                    raise RuntimeError("simplicial numerical gate failed; no performance or training launch")
        if on_gpu and not correctness_only:
            cases = [("global", (0, 0))]
            for w in WINDOW_PAIRS:
                cases += [("local", w), ("simplicial", w)]
            for kind, window in cases:
                bench = benchmark_case(kind, window, sequence=sequence, batch=batch, repetitions=repetitions)
                evidence["benchmarks"].append(bench)
                save()
                print(json.dumps({k: v for k, v in bench.items() if not k.endswith("_ms")} |
                                 {"median_forward_ms": sorted(bench["forward_ms"])[len(bench["forward_ms"]) // 2]}), flush=True)
        evidence["status"] = "passed"
    except Exception as error:
        evidence["status"], evidence["error"] = "failed", f"{type(error).__name__}: {error}"
        raise
    finally:
        evidence["ended_unix"] = time.time()
        save()
    return evidence


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--output", type=Path, required=True)
    ap.add_argument("--sequence", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--repetitions", type=int, default=20)
    ap.add_argument("--correctness-only", action="store_true")
    a = ap.parse_args(argv)
    try:
        run(a.output, sequence=a.sequence, batch=a.batch, repetitions=a.repetitions, correctness_only=a.correctness_only)
    except RuntimeError as error:
        print(f"preflight failed: {error}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
