"""The report card of one end-to-end pipeline run (tokenizer -> base model -> evaluation -> chat SFT -> RL).

Every stage calls ``report.log(section, [dict or text, ...])`` when it finishes; the section is stored twice: as markdown
(for people) and as JSON (for the summary, so that nothing has to be parsed back out of prose).  ``generate()`` stitches
the header and the sections in the pipeline's order into ``report.md`` and appends a summary: one table with the headline
metrics per stage (base / sft / rl) and the wall-clock time from ``reset()`` to the last non-experimental section.
``reset()`` starts a new card: it removes old sections and writes the header with what the run ran on (source commit and
dirtiness, host, Python / PyTorch versions, GPUs as PyTorch reports them).  Ranks other than 0 get a report that
ignores everything.  (Reference: src/archlab/speedrun/report.py:122-441.)
"""
from __future__ import annotations

import datetime
import json
import os
import platform
import socket
import subprocess
from pathlib import Path

STAGE_ORDER = ("tokenizer-training", "tokenizer-evaluation", "base-model-training", "base-model-loss", "base-model-evaluation", "chat-sft",
               "chat-evaluation-sft", "chat-rl", "chat-evaluation-rl")
SUMMARY = {"base-model-evaluation": ("base", ("CORE",)), "chat-evaluation-sft": ("sft", ("ARC-Easy", "ARC-Challenge", "MMLU", "GSM8K", "HumanEval", "ChatCORE")),
           "chat-evaluation-rl": ("rl", ("GSM8K",))}
EXPERIMENTAL = ("chat-rl", "chat-evaluation-rl")                 # not counted into the wall-clock time of the card
_STAMP = "%Y-%m-%d %H:%M:%S"


def slug(section: str) -> str:
    return section.lower().replace(" ", "-")


def _git(*args: str) -> str:
    try:
        return subprocess.run(["git", *args], capture_output=True, text=True, timeout=10, cwd=Path(__file__).resolve().parents[2]).stdout.strip()
    except (OSError, subprocess.TimeoutExpired):
        return ""


def environment() -> dict:
    import torch

    info = {"commit": _git("rev-parse", "--short", "HEAD") or "unknown", "dirty": bool(_git("status", "--porcelain")), "host": socket.gethostname(),
            "platform": platform.platform(), "python": platform.python_version(), "torch": torch.__version__, "cpus": os.cpu_count()}
    if torch.cuda.is_available():
        props = [torch.cuda.get_device_properties(i) for i in range(torch.cuda.device_count())]
        info["gpus"] = {"count": len(props), "names": sorted({p.name for p in props}), "total_memory_gib": round(sum(p.total_memory for p in props) / 2 ** 30, 1)}
    else:
        info["gpus"] = {"count": 0}
    return info


def _format(value) -> str:
    if isinstance(value, float):
        return f"{value:.4f}"
    if isinstance(value, int) and not isinstance(value, bool) and value >= 10_000:
        return f"{value:,}"
    return str(value)


class RunReport:
    def __init__(self, directory, *, clock=datetime.datetime.now):
        self.dir, self.clock = Path(directory), clock
        self.dir.mkdir(parents=True, exist_ok=True)

    def reset(self, env: dict | None = None) -> Path:
        for name in STAGE_ORDER:
            for suffix in (".md", ".json"):
                (self.dir / (name + suffix)).unlink(missing_ok=True)
        (self.dir / "report.md").unlink(missing_ok=True)
        env = environment() if env is None else env
        started = self.clock().strftime(_STAMP)
        lines = ["# Run report", "", "## Environment", ""] + [f"- {k}: {_format(v)}" for k, v in env.items()] + ["", f"Run started: {started}", "", "---", ""]
        (self.dir / "header.md").write_text("\n".join(lines))
        (self.dir / "header.json").write_text(json.dumps({"environment": env, "started": started}))
        return self.dir / "header.md"

    def log(self, section: str, data: list) -> Path:
        name, stamp = slug(section), self.clock().strftime(_STAMP)
        fields: dict = {}
        lines = [f"## {section}", f"timestamp: {stamp}", ""]
        for item in data:
            if not item:
                continue
            if isinstance(item, str):
                lines.append(item.rstrip("\n"))
            else:
                fields.update(item)
                lines += [f"- {k}: {_format(v)}" for k, v in item.items()]
        (self.dir / f"{name}.md").write_text("\n".join(lines) + "\n\n")
        (self.dir / f"{name}.json").write_text(json.dumps({"section": section, "timestamp": stamp, "fields": fields}, default=str))
        return self.dir / f"{name}.md"

    def generate(self) -> Path:
        out, metrics, end = [], {}, None
        header = self.dir / "header.md"
        start = None
        if header.exists():
            out.append(header.read_text())
            start = datetime.datetime.strptime(json.loads((self.dir / "header.json").read_text())["started"], _STAMP)
        else:
            out.append("# Run report\n\n(no header: the card was never reset)\n\n")
        missing = []
        for name in STAGE_ORDER:
            if not (self.dir / f"{name}.md").exists():
                missing.append(name)
                continue
            out.append((self.dir / f"{name}.md").read_text())
            body = json.loads((self.dir / f"{name}.json").read_text())
            if name not in EXPERIMENTAL:
                stamp = datetime.datetime.strptime(body["timestamp"], _STAMP)
                end = stamp if end is None else max(end, stamp)        # the latest one, whatever order stages were re-run in
            if name in SUMMARY:
                stage, keys = SUMMARY[name]
                metrics[stage] = {k: body["fields"][k] for k in keys if k in body["fields"]}
        names = sorted({k for m in metrics.values() for k in m}, key=lambda k: (k != "CORE", k == "ChatCORE", k))
        table = ["## Summary", "", f"| {'Metric':<15} | {'BASE':<8} | {'SFT':<8} | {'RL':<8} |", f"|{'-' * 17}|{'-' * 10}|{'-' * 10}|{'-' * 10}|"]
        for k in names:
            table.append(f"| {k:<15} | " + " | ".join(f"{_format(metrics.get(s, {}).get(k, '-')):<8}" for s in ("base", "sft", "rl")) + " |")
        if start and end:
            seconds = int((end - start).total_seconds())
            table += ["", f"Total wall clock time: {seconds // 3600}h{seconds % 3600 // 60}m"]
        else:
            table += ["", "Total wall clock time: unknown"]
        if missing:
            table += ["", "Sections not run: " + ", ".join(missing)]
        path = self.dir / "report.md"
        path.write_text("".join(out) + "\n".join(table) + "\n")
        return path


class NullReport:
    def log(self, *args, **kwargs):
        return None

    def reset(self, *args, **kwargs):
        return None

    def generate(self, *args, **kwargs):
        return None


def get_report(directory, rank: int | None = None):
    rank = int(os.environ.get("RANK", "0")) if rank is None else rank
    return RunReport(directory) if rank == 0 else NullReport()
