"""A supervised bootstrap experiment (assistant-only cross entropy from an exported parent): a typed recipe, the
settings it may and may not change, and the asset checks that bind parent, tokenizer and data together before launch.

Recipe (YAML): ``name``, ``parent_checkpoint`` (an export directory), ``data_manifest`` (prepared agent-trajectory
data), ``parent_stage`` (``original_base`` | ``package_sft``), ``variant`` (``normal`` | ``simplicial``), ``objective``
(only ``assistant_ce``), ``native_context`` and free-form ``settings`` applied over the trainer defaults
(``key=value`` overrides address both levels, ``settings.<dotted.key>=...``).

``validate_settings`` keeps the experiment what it says it is: full weights from exactly the declared parent, data
parallelism only, one un-padded sequence per micro-batch and no truncation (over-long rows are a data error), the
prepared-trajectory dataset, bf16 with a sharded Adam, a fresh start.  ``validate_assets`` reads files only: the parent
export's receipt verifies and its conversion state equals the declared variant; the data manifest is of the prepared
format, its tokenizer and template hashes equal the parent export's files, its EOS / mask-alignment / context agree with
the settings, its split files hash as recorded and are the ones the settings point to, and there is at least one
complete global batch.  ``source_snapshot`` / ``verify_source`` freeze the package sources the run was validated with;
receipts are written once and never rewritten differently.  (Reference: src/archlab/training/bootstrap.py:27-300.)
"""
from __future__ import annotations

import copy
import hashlib
import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any

import yaml

from ..ckpt.formats import verify_hf_export
from ..contracts.substrate import sha256_file

PARENT_STAGES = ("original_base", "package_sft")
DATA_FORMAT = "archlab.prepared-agentic-sft.v1"
DEFAULT_SETTINGS = {
    "model": {"path": None, "lora_rank": 0, "override_config": {}},
    "engine": {"dtype": "bfloat16", "tensor_parallel": 1, "pipeline_parallel": 1, "context_parallel": 1, "expert_parallel": 1,
               "sharded_optimizer": True, "sequence_packing": False},
    "data": {"dataset": "archlab_b200.data.agentic_sft:PreparedTrajectories", "train_files": [], "val_files": [], "max_length": 131072,
             "micro_batch_size_per_gpu": 1, "train_batch_size": 8, "pad_mode": "no_padding", "truncation": "error"},
    "trainer": {"nnodes": 1, "gpus_per_node": 8, "resume_mode": "disable", "experiment_name": None},
}


@dataclass
class BootstrapExperiment:
    name: str
    parent_checkpoint: str
    data_manifest: str
    parent_stage: str = "original_base"
    variant: str = "simplicial"
    objective: str = "assistant_ce"
    native_context: int = 131072
    settings: dict[str, Any] = field(default_factory=dict)


def _set(tree: dict, dotted: str, value) -> None:
    *parents, leaf = dotted.split(".")
    for key in parents:
        tree = tree.setdefault(key, {})
    tree[leaf] = value


def read_bootstrap(path, overrides: list[str] = ()) -> BootstrapExperiment:
    body = yaml.safe_load(Path(path).read_text())
    unknown = set(body) - set(BootstrapExperiment.__dataclass_fields__)
    if unknown:
        raise ValueError(f"unknown bootstrap recipe keys: {sorted(unknown)}")
    body.setdefault("settings", {})
    for override in overrides:
        key, sep, raw = override.partition("=")
        if not sep or not key:
            raise ValueError("overrides must use key=value")
        value = yaml.safe_load(raw)
        if key.startswith("settings."):
            body["settings"][key.removeprefix("settings.")] = value
        elif key in BootstrapExperiment.__dataclass_fields__ and key != "settings":
            body[key] = value
        else:
            raise ValueError(f"unknown bootstrap override: {key}")
    try:
        experiment = BootstrapExperiment(**body)
    except TypeError as missing:
        raise ValueError(f"incomplete bootstrap recipe: {missing}") from missing
    if experiment.objective != "assistant_ce":
        raise ValueError("a bootstrap uses assistant-only cross entropy")
    if experiment.variant not in ("normal", "simplicial") or experiment.parent_stage not in PARENT_STAGES:
        raise ValueError("a bootstrap needs a normal or simplicial export of a known parent stage")
    if type(experiment.native_context) is not int or experiment.native_context <= 0:
        raise ValueError("native_context must be a positive integer")
    return experiment


def compose_settings(experiment: BootstrapExperiment) -> dict:
    config = copy.deepcopy(DEFAULT_SETTINGS)
    for dotted, value in experiment.settings.items():
        section = dotted.split(".")[0]
        if section not in config:
            raise ValueError(f"unknown settings section: {section}")
        _set(config, dotted, value)
    config["trainer"]["experiment_name"] = experiment.name
    validate_settings(experiment, config)
    return config


def validate_settings(experiment: BootstrapExperiment, config: dict) -> None:
    model, engine, data, trainer = (config[k] for k in ("model", "engine", "data", "trainer"))
    if model["path"] != experiment.parent_checkpoint:
        raise ValueError("a bootstrap starts from its explicit parent export")
    if model.get("lora_rank") or model.get("override_config"):
        raise ValueError("a bootstrap trains full weights on the unchanged exported geometry")
    if engine["dtype"] != "bfloat16" or not engine["sharded_optimizer"]:
        raise ValueError("a bootstrap uses bf16 with a sharded Adam")
    if any(engine[k] != 1 for k in ("tensor_parallel", "pipeline_parallel", "context_parallel", "expert_parallel")):
        raise ValueError("a bootstrap supports data parallelism only")
    if engine["sequence_packing"] or data["pad_mode"] != "no_padding" or data["truncation"] != "error":
        raise ValueError("a bootstrap feeds one un-padded, un-truncated sequence per micro-batch")
    world = trainer["nnodes"] * trainer["gpus_per_node"]
    if data["micro_batch_size_per_gpu"] != 1 or data["train_batch_size"] < world or data["train_batch_size"] % world:
        raise ValueError("the global batch must be a whole number of one-sequence micro-batches per GPU")
    if not 0 < data["max_length"] <= experiment.native_context:
        raise ValueError("max_length must lie inside the model's native context")
    if data["dataset"] != DEFAULT_SETTINGS["data"]["dataset"]:
        raise ValueError("a bootstrap requires prepared assistant masks")
    if trainer["resume_mode"] != "disable":
        raise ValueError("a bootstrap starts a fresh experiment")


def validate_assets(experiment: BootstrapExperiment, config: dict) -> dict:
    root = Path(experiment.parent_checkpoint)
    exported = json.loads((root / "config.json").read_text())
    converted = bool(exported.get("conversion"))
    if converted != (experiment.variant == "simplicial"):
        raise ValueError("the export's conversion state differs from the bootstrap's variant")
    if exported.get("trainable_mode", "full") != "full" or (converted and exported.get("adapter")):
        raise ValueError("a bootstrap requires a full-weight export without adapters")
    receipt = verify_hf_export(root)
    lineage = receipt.get("lineage", {})
    if experiment.parent_stage == "package_sft":
        if lineage.get("stage") != "package_sft" or not lineage.get("supervised_tokens") or lineage.get("parent_state_sha256") == receipt["state_sha256"]:
            raise ValueError("the package-SFT parent does not establish trained weights")
    elif lineage.get("stage") not in (None, "original_base", "conversion"):
        raise ValueError("an original-base bootstrap cannot start from a trained export")
    manifest_path = Path(experiment.data_manifest)
    manifest = json.loads(manifest_path.read_text())
    if manifest.get("format") != DATA_FORMAT:
        raise ValueError("a bootstrap requires a prepared agentic SFT manifest")
    tok = manifest["tokenization"]
    if tok.get("loss_mask_alignment") != "unshifted-target-token" or tok.get("max_length") != config["data"]["max_length"]:
        raise ValueError("prepared mask alignment or context differs from the settings")
    if tok.get("generation_eos_token_id") != exported.get("eos_token_id"):
        raise ValueError("prepared EOS differs from the exported model's")
    for name, expected in tok["files"].items():
        if Path(name).name != name or not (root / name).is_file() or sha256_file(root / name) != expected:
            raise ValueError(f"prepared tokenizer / template checksum differs: {name}")
    if not {"tokenizer.json"} <= tok["files"].keys():
        raise ValueError("the prepared manifest does not pin the tokenizer")
    for split in ("train", "validation"):
        item = manifest["files"][split]
        target = manifest_path.parent / item["name"]
        if Path(item["name"]).name != item["name"] or sha256_file(target) != item["sha256"]:
            raise ValueError(f"prepared data checksum mismatch: {split}")
        files = config["data"]["train_files" if split == "train" else "val_files"]
        if [str(Path(f).resolve()) for f in files] != [str(target.resolve())]:
            raise ValueError(f"the settings' data files differ from the prepared manifest: {split}")
    if manifest["files"]["train"]["rows"] < config["data"]["train_batch_size"]:
        raise ValueError("the data cannot provide one complete global batch")
    return {"export_receipt_sha256": sha256_file(root / "EXPORT.json"), "state_sha256": receipt["state_sha256"],
            "data_manifest_sha256": sha256_file(manifest_path), "parent_stage": experiment.parent_stage, "variant": experiment.variant,
            "conversion": exported.get("conversion"), "supervision": manifest.get("supervision")}


def source_snapshot(package_root, recipe) -> dict:
    paths = sorted({*Path(package_root).rglob("*.py"), Path(recipe).resolve()})
    files = {str(p.resolve()): sha256_file(p) for p in paths}
    return {"sha256": hashlib.sha256(json.dumps(files, sort_keys=True).encode()).hexdigest(), "files": files}


def verify_source(snapshot: dict) -> None:
    for name, expected in snapshot["files"].items():
        if sha256_file(name) != expected:
            raise ValueError(f"bootstrap source changed after the freeze: {name}")


def write_once(path, text: str) -> None:
    path = Path(path)
    if path.exists():
        if path.read_text() != text:
            raise ValueError(f"an immutable bootstrap receipt already differs: {path}")
        return
    with path.open("x") as f:
        f.write(text)


def prepare(recipe, output, overrides: list[str] = (), *, package_root=None) -> dict:
    """Resolve, validate and freeze; writes ``bootstrap.json`` (once) and returns it.  Launching is the caller's step."""
    experiment = read_bootstrap(recipe, list(overrides))
    config = compose_settings(experiment)
    assets = validate_assets(experiment, config)
    snapshot = source_snapshot(package_root or Path(__file__).resolve().parents[1], recipe)
    receipt = {"experiment": asdict(experiment), "settings": config, "assets": assets, "source_sha256": snapshot["sha256"]}
    Path(output).mkdir(parents=True, exist_ok=True)
    write_once(Path(output) / "bootstrap.json", json.dumps(receipt, indent=1, sort_keys=True) + "\n")
    write_once(Path(output) / "source_snapshot.json", json.dumps(snapshot, indent=1, sort_keys=True) + "\n")
    return receipt
