"""On-disk checkpoint and export layouts that downstream export / serving-conversion code reads.

* Megatron legacy ``torch``: ``latest_checkpointed_iteration.txt`` + ``iter_{it:07d}/mp_rank_XX/
  model_optim_rng.pt`` (src/archlab/megatron/train.py:350-376).
* Megatron ``torch_dist``: ``iter_{it:07d}/{.metadata, common.pt, *.distcp}`` written through
  ``torch.distributed.checkpoint``; required key families ``embedding.* / decoder.*``,
  ``optimizer.*`` with ``exp_avg`` / ``exp_avg_sq``, ``rng_state*`` (megatron/export_eval.py:32-84).
* HF export: ``config.json`` + ``model.safetensors`` + ``EXPORT.json{format, state_sha256, files}``
  (src/archlab/training/limite.py:329-369).
* V4.1 full-sharded-v1: ``COMPLETE.json`` + ``rank-XX/MANIFEST.json`` with per-tensor chunk lists and
  hashes; layouts ``replicated`` / ``row{W}`` / ``expert_ep{E}_fsdp{F}``
  (src/archlab/serving/v41_checkpoint_inventory.py:26-135).
* V4.1 released-name export: one tensor per ``tensor-NNNNNN.safetensors``, index + manifest,
  ``EXPORT_COMPLETE.json`` written last (src/archlab/serving/v41_export.py:27-295).
* Run receipts: ``RUNNING.json`` -> ``COMPLETE.json`` / ``FAILED.json`` (megatron/train.py:396-422).
"""
from __future__ import annotations

import hashlib
import json
import math
import re
import shutil
import time
from collections import Counter
from pathlib import Path
from typing import Any

import torch

from ..contracts.substrate import atomic_write_json, sha256_file

_BYTES = {"torch.float32": 4, "torch.bfloat16": 2, "torch.float16": 2, "torch.float8_e4m3fn": 1, "torch.int8": 1,
          "torch.int32": 4, "torch.int64": 8, "torch.uint8": 1}


# ------------------------------------------------------------------------------------------------
# Megatron layouts
# ------------------------------------------------------------------------------------------------
def _tracker(root: Path) -> Path:
    return root / "latest_checkpointed_iteration.txt"


def save_megatron_torch(root, iteration: int, model_state: dict, optimizer_state: dict | None = None, *, tp_rank: int = 0,
                        pp_rank: int | None = None, rng_state=None, args: dict | None = None) -> Path:
    root = Path(root)
    sub = f"mp_rank_{tp_rank:02d}" + (f"_{pp_rank:03d}" if pp_rank is not None else "")
    d = root / f"iter_{iteration:07d}" / sub
    d.mkdir(parents=True, exist_ok=True)
    payload = {"iteration": iteration, "model": model_state, "checkpoint_version": 3.0, "args": args or {}}
    if optimizer_state is not None:
        payload["optimizer"] = optimizer_state
    if rng_state is not None:
        payload["rng_state"] = rng_state
    tmp = d / "model_optim_rng.pt.tmp"
    torch.save(payload, tmp)
    tmp.replace(d / "model_optim_rng.pt")
    _tracker(root).write_text(str(iteration))
    return d / "model_optim_rng.pt"


def latest_iteration(root) -> int:
    text = _tracker(Path(root)).read_text().strip()
    if not text.isdigit():
        raise ValueError(f"checkpoint tracker does not name an iteration: {text!r}")
    return int(text)


def validate_megatron_torch(root, *, require_optimizer: bool = True) -> dict:
    root = Path(root)
    it = latest_iteration(root)
    files = sorted((root / f"iter_{it:07d}").glob("**/model_optim_rng.pt"))
    if not files:
        raise FileNotFoundError(f"no model_optim_rng.pt under iter_{it:07d}")
    for f in files:
        payload = torch.load(f, map_location="cpu", weights_only=False)
        if payload.get("iteration") != it or "model" not in payload:
            raise ValueError(f"{f} does not hold iteration {it}")
        if require_optimizer and "optimizer" not in payload:
            raise ValueError(f"{f} has no optimizer state")
    return {"format": "torch", "iteration": it, "shards": len(files)}


def save_megatron_dist(root, iteration: int, model_state: dict, optimizer_state: dict | None = None, rng_state=None,
                       common: dict | None = None) -> Path:
    """``torch_dist`` layout through torch.distributed.checkpoint (single- or multi-process)."""
    import torch.distributed.checkpoint as dcp

    root = Path(root)
    d = root / f"iter_{iteration:07d}"
    d.mkdir(parents=True, exist_ok=True)
    flat = {f"{k}": v for k, v in model_state.items()}
    for name, st in (optimizer_state or {}).items():
        for key, val in st.items():
            flat[f"optimizer.state.{key}.{name}"] = val
    if rng_state is not None:
        flat["rng_state.0"] = rng_state if isinstance(rng_state, torch.Tensor) else torch.as_tensor(bytearray(json.dumps(rng_state).encode()))
    dcp.save(flat, checkpoint_id=str(d))
    torch.save({"iteration": iteration, **(common or {})}, d / "common.pt")
    _tracker(root).write_text(str(iteration))
    return d


def validate_megatron_dist(root) -> dict:
    import torch.distributed.checkpoint as dcp

    root = Path(root)
    it = latest_iteration(root)
    d = root / f"iter_{it:07d}"
    if not (d / ".metadata").is_file() or not (d / "common.pt").is_file() or not list(d.glob("*.distcp")):
        raise FileNotFoundError("torch_dist checkpoint needs .metadata, common.pt and *.distcp files")
    keys = list(dcp.FileSystemReader(str(d)).read_metadata().state_dict_metadata)
    has = lambda pat: any(re.search(pat, k) for k in keys)
    if not (has(r"^(module\.)?(embedding|decoder)\.")):
        raise ValueError("no embedding.* / decoder.* model keys")
    missing = [p for p in (r"^optimizer\..*exp_avg\.", r"^optimizer\..*exp_avg_sq\.", r"^rng_state") if not has(p)]
    if missing:
        raise ValueError(f"torch_dist checkpoint lacks key families: {missing}")
    return {"format": "torch_dist", "iteration": it, "keys": len(keys)}


def load_megatron_dist(root, template: dict) -> dict:
    import torch.distributed.checkpoint as dcp

    root = Path(root)
    dcp.load(template, checkpoint_id=str(root / f"iter_{latest_iteration(root):07d}"))
    return template


# ------------------------------------------------------------------------------------------------
# HF safetensors export
# ------------------------------------------------------------------------------------------------
def state_sha256(state: dict[str, torch.Tensor]) -> str:
    digest = hashlib.sha256()
    for name in sorted(state):
        t = state[name].detach().contiguous().cpu()
        digest.update(json.dumps({"name": name, "shape": list(t.shape), "dtype": str(t.dtype)}, sort_keys=True).encode())
        digest.update(bytes(t.view(torch.uint8).untyped_storage()) if t.numel() else b"")
    return digest.hexdigest()


def export_hf(out_dir, state: dict[str, torch.Tensor], config: dict, *, export_format: str = "archlab-hf-v1",
              extra_files: dict[str, bytes] | None = None, lineage: dict | None = None,
              tokenizer_dir=None, tokenizer_identity_sha256: str | None = None) -> dict:
    """Writes config.json + model.safetensors (+ assets), then EXPORT.json last, then re-loads to verify.

    ``tokenizer_dir``: the tokenizer's files (``TOKENIZER_ASSETS``, those that exist) are copied beside the weights so
    the export loads on its own; ``tokenizer.json`` or a sentencepiece model must be among them.  Their combined digest
    (``tokenizer_identity``) goes into the receipt and must equal ``tokenizer_identity_sha256`` when that is given, so a
    checkpoint is never shipped with another run's vocabulary (src/archlab/training/sft_export.py:24-40,219-244).
    """
    from safetensors.torch import load_file, save_file

    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    identity = None
    if tokenizer_dir is not None:
        identity = tokenizer_identity(tokenizer_dir)
        if tokenizer_identity_sha256 is not None and identity != tokenizer_identity_sha256:
            raise ValueError("the tokenizer directory is not the tokenizer the checkpoint was trained with")
        vocab = config.get("vocab_size")
        size = tokenizer_vocab_size(tokenizer_dir)
        if vocab is not None and size is not None and size > vocab:
            raise ValueError(f"tokenizer has {size} entries, the model's embedding only {vocab}")
        for name in _present_assets(tokenizer_dir):
            shutil.copyfile(Path(tokenizer_dir) / name, out / name)
    tensors = {k: v.detach().contiguous().cpu() for k, v in state.items()}
    (out / "config.json").write_text(json.dumps(config, indent=2, sort_keys=True))
    save_file(tensors, str(out / "model.safetensors"), metadata={"format": "pt"})
    for name, data in (extra_files or {}).items():
        if Path(name).name != name:
            raise ValueError("asset names must be basenames")
        (out / name).write_bytes(data)
    back = load_file(str(out / "model.safetensors"))
    digest = state_sha256(tensors)
    if state_sha256(back) != digest:
        raise RuntimeError("exported weights do not round-trip")
    files = {p.name: {"bytes": p.stat().st_size, "sha256": sha256_file(p)} for p in sorted(out.iterdir())
             if p.is_file() and p.name != "EXPORT.json"}
    receipt = {"format": export_format, "state_sha256": digest, "files": files, "tensor_count": len(tensors),
               "lineage": lineage or {}}
    if identity is not None:
        receipt["tokenizer_identity_sha256"] = identity
    atomic_write_json(out / "EXPORT.json", receipt)
    return receipt


TOKENIZER_ASSETS = ("tokenizer.json", "tokenizer.model", "tokenizer_config.json", "special_tokens_map.json", "added_tokens.json",
                    "vocab.json", "merges.txt", "chat_template.jinja", "generation_config.json")


def _present_assets(directory) -> list[str]:
    names = [n for n in TOKENIZER_ASSETS if (Path(directory) / n).is_file()]
    if not {"tokenizer.json", "tokenizer.model"} & set(names):
        raise ValueError("a tokenizer directory needs tokenizer.json or tokenizer.model")
    return names


def tokenizer_identity(directory) -> str:
    """One digest over the names and contents of the tokenizer's files, independent of where they are stored."""
    h = hashlib.sha256()
    for name in _present_assets(directory):
        h.update(name.encode() + b"\0" + bytes.fromhex(sha256_file(Path(directory) / name)))
    return h.hexdigest()


def tokenizer_vocab_size(directory) -> int | None:
    """Highest token id + 1 of a ``tokenizer.json`` (vocabulary and added tokens); None for other tokenizer kinds."""
    path = Path(directory) / "tokenizer.json"
    if not path.is_file():
        return None
    body = json.loads(path.read_text())
    ids = [*body.get("model", {}).get("vocab", {}).values()] if isinstance(body.get("model", {}).get("vocab"), dict) else []
    ids += [t["id"] for t in body.get("added_tokens", [])]
    return max(ids) + 1 if ids else None


COPY_MARKER = "EXPORT_COPY_COMPLETE.json"


def valid_hf_export(path) -> bool:
    """What a loader needs at least: configuration, tokenizer and weights."""
    path = Path(path)
    return (path / "config.json").is_file() and ((path / "tokenizer.json").is_file() or (path / "tokenizer.model").is_file()) and (
        any(path.glob("*.safetensors")) or any(path.glob("pytorch_model*.bin")))


def copy_export(source, output) -> dict:
    """Copies a complete export to storage that supports neither rename nor metadata copies (object-store mounts): plain
    file copies, each re-hashed at the destination, then ``EXPORT_COPY_COMPLETE.json`` LAST with the per-file manifest.  A
    destination that is valid and carries the marker is left alone; one without the marker is copied again
    (src/archlab/megatron/export_eval.py:112-139)."""
    source, output = Path(source), Path(output)
    marker = output / COPY_MARKER
    if valid_hf_export(output) and marker.is_file():
        return json.loads(marker.read_text())
    if not valid_hf_export(source):
        raise RuntimeError(f"the source export is incomplete: {source}")
    output.mkdir(parents=True, exist_ok=True)
    manifest = []
    for src in sorted(f for f in source.rglob("*") if f.is_file()):
        rel = src.relative_to(source)
        dst = output / rel
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(src, dst)
        digest = sha256_file(src)
        if sha256_file(dst) != digest:
            raise RuntimeError(f"export copy hash mismatch: {rel}")
        manifest.append({"path": str(rel), "bytes": src.stat().st_size, "sha256": digest})
    if not valid_hf_export(output):
        raise RuntimeError(f"the copied export is incomplete: {output}")
    body = {"source": str(source), "files": manifest}
    marker.write_text(json.dumps(body, sort_keys=True) + "\n")
    return body


def verify_hf_export(out_dir) -> dict:
    from safetensors.torch import load_file

    out = Path(out_dir)
    receipt = json.loads((out / "EXPORT.json").read_text())
    for name, meta in receipt["files"].items():
        p = out / name
        if not p.is_file() or p.stat().st_size != meta["bytes"] or sha256_file(p) != meta["sha256"]:
            raise ValueError(f"export file changed: {name}")
    if state_sha256(load_file(str(out / "model.safetensors"))) != receipt["state_sha256"]:
        raise ValueError("export state digest mismatch")
    return receipt


# ------------------------------------------------------------------------------------------------
# V4.1 fully sharded training checkpoint
# ------------------------------------------------------------------------------------------------
V41_FORMAT = "archlab-v41-full-sharded-v1"
_EXPERT_SUFFIXES = (".ffn.experts.gate_and_up_projs", ".ffn.experts.down_projs")


def shard_extent(size: int, pieces: int, index: int) -> tuple[int, int]:
    """(offset, length) of piece ``index`` of an axis of ``size`` cut into ``pieces``.

    The on-disk layout fixes the rule (src/archlab/serving/v41_checkpoint_inventory.py:20-23): every
    piece is ``ceil(size / pieces)`` wide, the last non-empty one takes what is left and pieces past
    the end are empty (offset = size, length 0).  10 rows over 4 pieces: (0,3) (3,3) (6,3) (9,1).
    """
    width = -(-size // pieces)
    offset = min(index * width, size)
    return offset, min(width, size - offset)


def _placement(name: str, shape: list[int], rank: int, world: int, ep: int, fsdp: int):
    off, ext = [0] * len(shape), list(shape)
    axes = [(0, ep, rank % ep), (1, fsdp, rank // ep)] if name.endswith(_EXPERT_SUFFIXES) else [(0, world, rank)]
    for axis, pieces, idx in axes:
        off[axis], ext[axis] = shard_extent(shape[axis], pieces, idx)
    return off, ext


def write_v41_sharded(root, state: dict[str, torch.Tensor], *, cursor: dict, world_size: int = 16, ep_size: int = 8,
                      expert_fsdp_size: int = 2, engram_owners: int = 16, variant: str = "normal",
                      replicated: set[str] | None = None, chunk_elements: int = 1 << 24) -> dict:
    """Single-process writer of the layout every rank would produce (tests, conversions)."""
    root = Path(root)
    contract = {"world_size": world_size, "ep_size": ep_size, "expert_fsdp_size": expert_fsdp_size,
                "engram_owners": engram_owners, "all_parameters_unfrozen": True, "variant": variant}
    replicated = replicated or set()
    for rank in range(world_size):
        d = root / f"rank-{rank:02d}"
        d.mkdir(parents=True, exist_ok=True)
        tensors = []
        for i, (name, t) in enumerate(state.items()):
            t = t.detach().cpu()
            if name in replicated or t.ndim == 0:
                local = t
            else:
                off, ext = _placement(name, list(t.shape), rank, world_size, ep_size, expert_fsdp_size)
                local = t[tuple(slice(o, o + e) for o, e in zip(off, ext))]
            flat = local.contiguous().view(-1)
            chunks = []
            for c, s0 in enumerate(range(0, max(flat.numel(), 1), chunk_elements)):
                piece = flat[s0:s0 + chunk_elements].clone()
                fname = f"t{i:05d}-c{c:03d}.pt"
                torch.save(piece, d / fname)
                chunks.append({"file": fname, "elements": piece.numel(),
                               "sha256": hashlib.sha256(piece.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()})
            tensors.append({"name": name, "global_shape": list(t.shape), "shape": list(local.shape), "dtype": str(t.dtype),
                            "chunks": chunks})
        atomic_write_json(d / "MANIFEST.json", {"rank": rank, "world_size": world_size, "cursor": cursor, "contract": contract,
                                                "tensors": tensors})
    marker = {"format": V41_FORMAT, "world_size": world_size, "contract": contract, "cursor": cursor, "written": time.time()}
    atomic_write_json(root / "COMPLETE.json", marker)
    return marker


class V41CheckpointInventory:
    """Metadata-level validation of a sharded checkpoint and bounded reconstruction of single tensors."""

    def __init__(self, checkpoint):
        self.path = Path(checkpoint)
        self.marker = m = json.loads((self.path / "COMPLETE.json").read_text())
        c = m["contract"]
        self.world = W = m["world_size"]
        if m["format"] != V41_FORMAT or c["world_size"] != W or c["ep_size"] * c["expert_fsdp_size"] != W or not c["all_parameters_unfrozen"]:
            raise ValueError("unsupported full-training checkpoint contract")
        self.manifests = []
        for r in range(W):
            man = json.loads((self.path / f"rank-{r:02d}/MANIFEST.json").read_text())
            if man["rank"] != r or man["world_size"] != W or man["cursor"] != m["cursor"] or man["contract"] != c:
                raise ValueError("rank manifest differs from COMPLETE")
            self.manifests.append(man)
        names = [t["name"] for t in self.manifests[0]["tensors"]]
        if len(set(names)) != len(names):
            raise ValueError("duplicate tensor names")
        if any([t["name"] for t in man["tensors"]] != names for man in self.manifests):
            raise ValueError("rank tensor lists differ")
        self.entries = {n: [man["tensors"][i] for man in self.manifests] for i, n in enumerate(names)}
        self.layouts = {n: self._layout(e) for n, e in self.entries.items()}

    def _layout(self, entries):
        first, c, W = entries[0], self.marker["contract"], self.world
        name, shape = first["name"], first["global_shape"]
        for e in entries:
            if any(e[k] != first[k] for k in ("name", "global_shape", "dtype")):
                raise ValueError(f"rank tensor identity differs: {name}")
            if sum(ch["elements"] for ch in e["chunks"]) != math.prod(e["shape"]):
                raise ValueError(f"chunk elements do not cover local shape: {name}")
        if all(e["shape"] == shape for e in entries):
            sig = [[(ch["elements"], ch["sha256"]) for ch in e["chunks"]] for e in entries]
            if any(s != sig[0] for s in sig[1:]):
                raise ValueError(f"replicated tensor checksums disagree: {name}")
            return "replicated", [tuple(0 for _ in shape)] * W
        expert = name.endswith(_EXPERT_SUFFIXES)
        if expert and len(shape) != 3:
            raise ValueError("expert tensor must have three axes")
        offsets = []
        for r, e in enumerate(entries):
            off, ext = _placement(name, shape, r, W, c["ep_size"], c["expert_fsdp_size"])
            if e["shape"] != ext:
                raise ValueError(f"unsupported placement for {name} rank {r}: {e['shape']}")
            offsets.append(tuple(off))
        return (f"expert_ep{c['ep_size']}_fsdp{c['expert_fsdp_size']}" if expert else f"row{W}"), offsets

    def report(self) -> dict:
        sizes = Counter()
        for e in self.entries.values():
            sizes[e[0]["dtype"]] += math.prod(e[0]["global_shape"]) * _BYTES[e[0]["dtype"]]
        return {"checkpoint": str(self.path.resolve()), "cursor": self.marker["cursor"], "variant": self.marker["contract"]["variant"],
                "tensor_count": len(self.entries), "layouts": dict(Counter(k for k, _ in self.layouts.values())),
                "unique_tensor_bytes_by_dtype": dict(sizes), "unique_tensor_bytes": sum(sizes.values()),
                "metadata_validated": True, "all_payloads_verified": False, "engine_ready": False, "optimizer_included": False}

    def read_tensor(self, name: str, *, max_bytes: int = 512 * 2 ** 20) -> torch.Tensor:
        entries = self.entries[name]
        shape, dtype = entries[0]["global_shape"], entries[0]["dtype"]
        if math.prod(shape) * _BYTES[dtype] > max_bytes:
            raise ValueError("tensor exceeds reconstruction limit; streaming export required")
        out = torch.empty(shape, dtype=getattr(torch, dtype.removeprefix("torch.")))
        kind, offsets = self.layouts[name]
        for r in (range(1) if kind == "replicated" else range(self.world)):
            e = entries[r]
            local = torch.empty(e["shape"], dtype=out.dtype)
            flat, pos = local.view(-1), 0
            for ch in e["chunks"]:
                if Path(ch["file"]).name != ch["file"]:
                    raise ValueError("chunk filename must be a basename")
                v = torch.load(self.path / f"rank-{r:02d}" / ch["file"], map_location="cpu", weights_only=True)
                if (v.ndim != 1 or v.dtype != out.dtype or v.numel() != ch["elements"]
                        or hashlib.sha256(v.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest() != ch["sha256"]):
                    raise ValueError(f"checkpoint payload mismatch: {name}")
                flat[pos:pos + v.numel()].copy_(v)
                pos += v.numel()
            out[tuple(slice(o, o + s) for o, s in zip(offsets[r], local.shape))].copy_(local)
        return out


# ------------------------------------------------------------------------------------------------
# V4.1 released-name export
# ------------------------------------------------------------------------------------------------
_RENAMES = (("embed_tokens.", "embed."), ("lm_head.", "head."), ("hc_attn.proj", "hc_attn_fn"), ("hc_ffn.proj", "hc_ffn_fn"),
            ("attn.sink", "attn_sink"), ("e_score_correction_bias", "gate.bias"))


def released_name(name: str) -> str:
    for a, b in _RENAMES:
        name = name.replace(a, b)
    return name


def export_v41_released(out_dir, tensors, *, engram_row_block: int = 0) -> dict:
    """``tensors``: iterable of (name, tensor).  Expert banks ``...experts.gate_and_up_projs`` [E, C, 2I] are
    split and transposed into per-expert ``w1`` / ``w3`` ([I, C]); ``...down_projs`` [E, I, C] into ``w2`` ([C, I]).
    One tensor per file; the index, the manifest and finally EXPORT_COMPLETE.json are written after all tensors."""
    from safetensors.torch import save_file

    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    weight_map, lines, n = {}, [], 0

    def emit(key: str, t: torch.Tensor):
        nonlocal n
        fname = f"tensor-{n:06d}.safetensors"
        save_file({key: t.detach().contiguous().cpu()}, str(out / fname))
        weight_map[key] = fname
        lines.append({"name": key, "file": fname, "shape": list(t.shape), "dtype": str(t.dtype), "sha256": sha256_file(out / fname)})
        n += 1

    for name, t in tensors:
        key = released_name(name)
        if name.endswith(".experts.gate_and_up_projs"):
            base = key.removesuffix("gate_and_up_projs")
            inter = t.shape[-1] // 2
            for e in range(t.shape[0]):
                emit(f"{base}{e}.w1.weight", t[e, :, :inter].t())
                emit(f"{base}{e}.w3.weight", t[e, :, inter:].t())
        elif name.endswith(".experts.down_projs"):
            base = key.removesuffix("down_projs")
            for e in range(t.shape[0]):
                emit(f"{base}{e}.w2.weight", t[e].t())
        elif engram_row_block and ".engram." in name and t.ndim == 2 and t.shape[0] > engram_row_block:
            for r0 in range(0, t.shape[0], engram_row_block):
                emit(f"{key}.rows.{r0}", t[r0:r0 + engram_row_block])
        else:
            emit(key, t)
    (out / "model.safetensors.index.json").write_text(json.dumps({"metadata": {"tensor_files": n}, "weight_map": weight_map}, indent=1))
    (out / "export-manifest.jsonl").write_text("".join(json.dumps(l) + "\n" for l in lines))
    done = {"format": "archlab-v41-released-names-v1", "tensors": n, "manifest_sha256": sha256_file(out / "export-manifest.jsonl")}
    atomic_write_json(out / "EXPORT_COMPLETE.json", done)
    return done


# ------------------------------------------------------------------------------------------------
# run receipts
# ------------------------------------------------------------------------------------------------
class RunReceipts:
    """RUNNING.json while the run is alive; afterwards COMPLETE.json, FAILED.json, or neither when the
    run was stopped on request (``stopped``)."""

    def __init__(self, run_dir, resolved: dict):
        self.dir = Path(run_dir)
        self.dir.mkdir(parents=True, exist_ok=True)
        if (self.dir / "COMPLETE.json").exists():
            raise FileExistsError("run directory already holds a completed run")
        atomic_write_json(self.dir / "resolved_run.json", resolved)
        atomic_write_json(self.dir / "RUNNING.json", {"started": time.time()})
        (self.dir / "FAILED.json").unlink(missing_ok=True)

    def log(self, record: dict) -> None:
        with open(self.dir / "metrics.jsonl", "a") as f:
            f.write(json.dumps(record) + "\n")

    def stopped(self, result: dict | None = None) -> None:
        """A requested stop before the step budget was used up: the partial result is recorded and
        RUNNING.json goes away, but no COMPLETE.json is written, so the directory can be resumed."""
        atomic_write_json(self.dir / "result.json", {**(result or {}), "outcome": "stopped"})
        (self.dir / "RUNNING.json").unlink(missing_ok=True)

    def finish(self, result: dict | None = None, error: BaseException | None = None) -> None:
        from ..contracts.substrate import classify_failure

        if error is None:
            atomic_write_json(self.dir / "result.json", result or {})
            atomic_write_json(self.dir / "COMPLETE.json", {"finished": time.time()})
        else:
            cls = classify_failure(error)
            atomic_write_json(self.dir / "FAILED.json", {"finished": time.time(), "error": repr(error),
                                                         "classification": cls.to_dict()})
        (self.dir / "RUNNING.json").unlink(missing_ok=True)
