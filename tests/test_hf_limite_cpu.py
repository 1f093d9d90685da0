"""The exported Limite directory loads through the stock Hugging Face entry points and reproduces the native logits."""
import json

import torch

from archlab_b200.models.limite import LimiteConfig, LimiteLM


def test_export_then_from_pretrained_reproduces_the_logits(tmp_path):
    from transformers import AutoConfig, AutoModelForCausalLM

    from archlab_b200.ckpt.formats import verify_hf_export
    from archlab_b200.serve import hf_limite

    torch.manual_seed(0)
    model = LimiteLM(LimiteConfig.tiny())
    model.init_weights()
    receipt = hf_limite.export_limite(tmp_path, model, lineage={"source": "unit test"})
    assert verify_hf_export(tmp_path)["state_sha256"] == receipt["state_sha256"]
    cfg = json.loads((tmp_path / "config.json").read_text())
    assert cfg["model_type"] == "archlab_limite" and cfg["architectures"] == ["ArchlabLimiteForCausalLM"]
    loaded_cfg = AutoConfig.from_pretrained(tmp_path)
    assert loaded_cfg.to_native() == model.config
    loaded = AutoModelForCausalLM.from_pretrained(tmp_path, dtype=torch.float32)
    ids = torch.randint(0, 128, (2, 12))
    with torch.no_grad():
        out = loaded(ids, labels=ids)
        torch.testing.assert_close(out.logits, model(ids), rtol=1e-5, atol=1e-5)
    want = model(ids[:, :-1], ids[:, 1:])
    torch.testing.assert_close(out.loss, want, rtol=1e-4, atol=1e-5)
    hf_limite.register()                                  # idempotent


def test_packaging_declares_the_console_scripts_and_the_plugin():
    import tomllib
    from pathlib import Path

    meta = tomllib.loads((Path(__file__).resolve().parents[1] / "pyproject.toml").read_text())
    assert meta["project"]["scripts"] == {"archlab": "archlab_b200.cli:main", "next-gen-arch": "archlab_b200.cli:main"}
    plug = meta["project"]["entry-points"]["vllm.general_plugins"]["archlab_limite"]
    module, func = plug.split(":")
    import importlib

    assert callable(getattr(importlib.import_module(module), func))
