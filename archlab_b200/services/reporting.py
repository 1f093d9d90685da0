"""Result tables and curves from run receipts: paired comparisons against a baseline, smoothed learning
curves, markdown tables (src/archlab/reporting/paired_curves.py, learning_curves.py, runs.py)."""
from __future__ import annotations

import json
import math
from pathlib import Path
from statistics import mean, median


def read_metrics(path) -> list[dict]:
    out = []
    for line in Path(path).read_text().splitlines():
        if line.strip():
            out.append(json.loads(line))
    return out


def learning_curve(rows: list[dict], key: str = "loss", *, ema: float = 0.0) -> list[tuple[int, float]]:
    pts, acc = [], None
    for r in rows:
        if key not in r or not math.isfinite(r[key]):
            continue
        acc = r[key] if acc is None or ema <= 0 else ema * acc + (1 - ema) * r[key]
        pts.append((int(r.get("step", len(pts) + 1)), acc))
    return pts


def final_value(rows: list[dict], key: str = "loss", *, tail: int = 10) -> float:
    vals = [r[key] for r in rows if key in r and math.isfinite(r[key])][-tail:]
    if not vals:
        raise ValueError(f"no finite {key!r} values")
    return mean(vals)


def paired_comparison(runs: dict[str, dict[int, float]], baseline: str) -> list[dict]:
    """``runs[variant][seed] = metric`` (lower is better).  Differences are taken seed by seed against the
    baseline so shared data-order noise cancels."""
    if baseline not in runs:
        raise ValueError("baseline variant missing")
    rows = []
    for variant, by_seed in sorted(runs.items()):
        seeds = sorted(set(by_seed) & set(runs[baseline]))
        if not seeds:
            continue
        diffs = [by_seed[s] - runs[baseline][s] for s in seeds]
        sd = (sum((d - mean(diffs)) ** 2 for d in diffs) / (len(diffs) - 1)) ** 0.5 if len(diffs) > 1 else float("nan")
        rows.append({"variant": variant, "seeds": len(seeds), "mean": mean(by_seed[s] for s in seeds), "delta_mean": mean(diffs),
                     "delta_median": median(diffs), "delta_sd": sd,
                     "wins": sum(d < 0 for d in diffs), "losses": sum(d > 0 for d in diffs)})
    return rows


def markdown_table(rows: list[dict], columns: list[str], *, digits: int = 4) -> str:
    fmt = lambda v: f"{v:.{digits}f}" if isinstance(v, float) else str(v)
    head = "| " + " | ".join(columns) + " |\n|" + "|".join("---" for _ in columns) + "|\n"
    return head + "".join("| " + " | ".join(fmt(r.get(c, "")) for c in columns) + " |\n" for r in rows)


# ======================================================================================================================
# Token-matched comparison of two training runs from their append-only ledgers
# (what the reference's paired report computes: src/archlab/reporting/runs.py:9-132, paired_curves.py:12-92)
# ======================================================================================================================
class TrainingLedger:
    """Validated rows of a run's ``train-metrics.jsonl`` (preceded by ``prior-phase-metrics.jsonl`` when present).

    A ledger is trusted only if its steps are contiguous, every row has a positive token count and a finite loss, and the
    cumulative token cursor equals the running sum of the rows' token counts.  A last line without its newline belongs to
    a writer that is still running and is left out; any other undecodable line is an error."""

    def __init__(self, rows: list[dict], sources: list[dict] | None = None):
        self.rows, self.sources = rows, sources or []
        self._validate()

    @staticmethod
    def decode(raw: bytes) -> list[dict]:
        rows, lines = [], raw.split(b"\n")                   # records are separated by LF only, never by Unicode separators
        for i, line in enumerate(lines):
            if not line.strip():
                continue
            try:
                row = json.loads(line)
            except json.JSONDecodeError:
                if i == len(lines) - 1 and not raw.endswith(b"\n"):
                    break
                raise
            if not isinstance(row, dict):
                raise ValueError("a training ledger holds JSON objects")
            rows.append(row)
        return rows

    @classmethod
    def read(cls, directory, *, include_history: bool = True) -> "TrainingLedger":
        import hashlib

        directory = Path(directory)
        files = [directory / "train-metrics.jsonl"]
        if include_history and (directory / "prior-phase-metrics.jsonl").exists():
            files.insert(0, directory / "prior-phase-metrics.jsonl")
        rows, sources = [], []
        for f in files:
            raw = f.read_bytes()
            part = cls.decode(raw)
            rows += part
            sources.append({"path": str(f.resolve()), "sha256": hashlib.sha256(raw).hexdigest(), "rows": len(part)})
        return cls(rows, sources)

    def _validate(self) -> None:
        if not self.rows:
            raise ValueError("empty training ledger")
        step = self.rows[0]["step"] - 1
        cursor = self.rows[0]["consumed_supervised_tokens"] - self.rows[0]["supervised_tokens"]
        if cursor < 0:
            raise ValueError("negative initial token cursor")
        for r in self.rows:
            if r["step"] != step + 1:
                raise ValueError("non-contiguous training steps")
            if r["supervised_tokens"] <= 0 or not math.isfinite(r["loss"]):
                raise ValueError("invalid token count or nonfinite loss")
            cursor += r["supervised_tokens"]
            if r["consumed_supervised_tokens"] != cursor:
                raise ValueError("token ledger differs from cumulative cursor")
            step = r["step"]

    @property
    def token_interval(self) -> tuple[int, int]:
        first, last = self.rows[0], self.rows[-1]
        return first["consumed_supervised_tokens"] - first["supervised_tokens"], last["consumed_supervised_tokens"]

    def window_mean(self, low: float, high: float) -> float:
        """Token-weighted mean loss over the token interval [low, high)."""
        if not (math.isfinite(low) and math.isfinite(high) and high > low):
            raise ValueError("token window must have finite increasing bounds")
        total = weight = 0.0
        for r in self.rows:
            end = r["consumed_supervised_tokens"]
            overlap = max(0, min(end, high) - max(end - r["supervised_tokens"], low))
            total, weight = total + overlap * r["loss"], weight + overlap
        if weight <= 0:
            raise ValueError("empty token window")
        return total / weight

    def smoothed(self, width: int) -> list[tuple[int, float]]:
        """(token cursor, token-weighted mean loss of the trailing ``width`` tokens) after every update."""
        if width <= 0:
            raise ValueError("smoothing token count must be positive")
        start = self.token_interval[0]
        return [(r["consumed_supervised_tokens"], self.window_mean(max(start, r["consumed_supervised_tokens"] - width), r["consumed_supervised_tokens"]))
                for r in self.rows]


PAIRED_FIELDS = ("consumed_supervised_tokens", "supervised_tokens", "input_tokens", "window_cursor", "learning_rate")


def matched_ledgers(first: TrainingLedger, second: TrainingLedger) -> tuple[TrainingLedger, TrainingLedger]:
    """The common steps of two runs, refusing pairs whose data or schedule cursors differ at a common step: updates are
    matched, never interpolated."""
    left, right = ({r["step"]: r for r in ledger.rows} for ledger in (first, second))
    steps = sorted(left.keys() & right.keys())
    if not steps:
        raise ValueError("runs have no common training steps")
    for s in steps:
        for f in PAIRED_FIELDS:
            if (f in left[s]) != (f in right[s]) or left[s].get(f) != right[s].get(f):
                raise ValueError(f"paired {f} differs at step {s}")
    return TrainingLedger([left[s] for s in steps]), TrainingLedger([right[s] for s in steps])


def paired_report(runs: dict[str, str], output, *, smoothing_tokens: int = 5_000_000, summary_tokens: int = 10_000_000,
                  current_phase_only: bool = False) -> dict:
    """Writes ``SUMMARY.json``, per-run snapshots and ``matched-training-curves.csv`` for exactly two labelled runs."""
    import csv

    from ..contracts.substrate import atomic_write_json

    if len(runs) != 2:
        raise ValueError("provide exactly two runs with distinct labels")
    if min(smoothing_tokens, summary_tokens) <= 0:
        raise ValueError("token windows must be positive")
    labels = list(runs)
    loaded = [TrainingLedger.read(runs[k], include_history=not current_phase_only) for k in labels]
    paired = matched_ledgers(*loaded)
    start, stop = paired[0].token_interval
    low = max(start, stop - summary_tokens)
    output = Path(output)
    output.mkdir(parents=True, exist_ok=False)
    summary = {"matched_steps": [paired[0].rows[0]["step"], paired[0].rows[-1]["step"]], "matched_token_interval": [start, stop],
               "summary_token_interval": [low, stop], "smoothing_tokens": smoothing_tokens, "runs": {}}
    for i, k in enumerate(labels):
        summary["runs"][k] = {"directory": str(Path(runs[k]).resolve()), "sources": loaded[i].sources, "latest_step": loaded[i].rows[-1]["step"],
                              "latest_tokens": loaded[i].rows[-1]["consumed_supervised_tokens"],
                              "matched_token_weighted_ce": paired[i].window_mean(low, stop)}
        (output / f"run-{i}-snapshot.jsonl").write_text("".join(json.dumps(r) + "\n" for r in loaded[i].rows))
    summary["first_minus_second_ce"] = (summary["runs"][labels[0]]["matched_token_weighted_ce"]
                                        - summary["runs"][labels[1]]["matched_token_weighted_ce"])
    atomic_write_json(output / "SUMMARY.json", summary, allow_nan=False)
    curves = [dict(p.smoothed(smoothing_tokens)) for p in paired]
    with (output / "matched-training-curves.csv").open("w", newline="") as f:
        w = csv.writer(f)
        w.writerow(["step", "supervised_tokens", *labels, *(f"{k}_smoothed" for k in labels)])
        for a, b in zip(paired[0].rows, paired[1].rows):
            t = a["consumed_supervised_tokens"]
            w.writerow([a["step"], t, a["loss"], b["loss"], curves[0][t], curves[1][t]])
    return summary


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(description="Summarise two token-matched training runs.")
    ap.add_argument("--run", nargs=2, action="append", required=True, metavar=("LABEL", "DIRECTORY"))
    ap.add_argument("--output", type=Path, required=True)
    ap.add_argument("--smoothing-tokens", type=int, default=5_000_000)
    ap.add_argument("--summary-tokens", type=int, default=10_000_000)
    ap.add_argument("--current-phase-only", action="store_true")
    a = ap.parse_args(argv)
    if len({label for label, _ in a.run}) != len(a.run):
        ap.error("run labels must be distinct")
    print(json.dumps(paired_report(dict(a.run), a.output, smoothing_tokens=a.smoothing_tokens, summary_tokens=a.summary_tokens,
                                   current_phase_only=a.current_phase_only), indent=2))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())


# ---- runs with different batch sizes on one token axis ---------------------------------------------------------------
def token_blocks(rows: list[dict], *, tokens_per_step: int, block_tokens: int, key: str = "loss") -> list[dict]:
    """Means of ``key`` over COMPLETE blocks of ``block_tokens`` consumed tokens.  Two runs whose optimizer steps hold
    different numbers of tokens become comparable point by point; a block with a missing step is left out rather than
    averaged over fewer steps.  (The reference aligns TensorBoard scalars the same way:
    src/archlab/reporting/learning_curves.py:16-50; here the source is the run's ``metrics.jsonl``.)"""
    if block_tokens % tokens_per_step:
        raise ValueError("a comparison block must hold a whole number of optimizer steps")
    per_block = block_tokens // tokens_per_step
    by_step = {int(r["step"]): r for r in rows if key in r and math.isfinite(r[key])}
    if not by_step:
        raise ValueError("no finite measurements")
    points = []
    for block in range(1, max(by_step) // per_block + 1):
        steps = range((block - 1) * per_block + 1, block * per_block + 1)
        if all(s in by_step for s in steps):
            points.append({"block": block, "step": steps[-1], "tokens": block * block_tokens,
                           key: sum(by_step[s][key] for s in steps) / per_block})
    if not points:
        raise ValueError("no complete token blocks")
    return points


def trailing_means(values: list[float], window: int) -> list[float]:
    return [sum(values[max(0, i + 1 - window):i + 1]) / (i + 1 - max(0, i + 1 - window)) for i in range(len(values))]


def aligned_curves(runs: dict[str, tuple[list[dict], int]], *, block_tokens: int, smoothing_blocks: int = 20, key: str = "loss") -> dict:
    """``runs``: label -> (ledger rows, tokens per optimizer step).  Returns per label the block means and their trailing
    mean, plus the differences against the first label at every token count all runs reached."""
    curves = {}
    for label, (rows, tokens_per_step) in runs.items():
        points = token_blocks(rows, tokens_per_step=tokens_per_step, block_tokens=block_tokens, key=key)
        smooth = trailing_means([p[key] for p in points], smoothing_blocks)
        curves[label] = [{**p, "smoothed": s} for p, s in zip(points, smooth)]
    first, *others = list(curves)
    base = {p["tokens"]: p for p in curves[first]}
    differences = {label: [{"tokens": p["tokens"], "delta": p[key] - base[p["tokens"]][key], "delta_smoothed": p["smoothed"] - base[p["tokens"]]["smoothed"]}
                           for p in curves[label] if p["tokens"] in base] for label in others}
    return {"block_tokens": block_tokens, "smoothing_blocks": smoothing_blocks, "curves": curves, "differences_against": first, "differences": differences}
