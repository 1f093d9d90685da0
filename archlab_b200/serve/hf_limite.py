"""Hugging Face boundary of the Limite family: ``AutoConfig`` / ``AutoModelForCausalLM`` resolve the model type
``archlab_limite`` to this package's decoder, so an exported directory (``ckpt.formats.export_hf``) loads with the stock
``from_pretrained`` call and hands back the same logits as ``models.limite.LimiteLM``
(the reference registers its decoder the same way: src/archlab/training/limite.py:73-374).

Importing this module performs the registration (idempotent).  ``register`` is also the vLLM general-plugin entry
point declared in ``pyproject.toml``: each serving process calls it, and when vLLM is importable the architecture
name is added to its model registry as well.
"""
from __future__ import annotations

from dataclasses import asdict, fields

import torch
from transformers import AutoConfig, AutoModelForCausalLM, PretrainedConfig, PreTrainedModel
from transformers.modeling_outputs import CausalLMOutput

from ..models.limite import LimiteConfig, LimiteLM

MODEL_TYPE = "archlab_limite"
ARCHITECTURE = "ArchlabLimiteForCausalLM"
_FIELDS = tuple(f.name for f in fields(LimiteConfig))


class LimiteHFConfig(PretrainedConfig):
    model_type = MODEL_TYPE

    def __init__(self, **kwargs):
        defaults = asdict(LimiteConfig())
        for name in _FIELDS:
            setattr(self, name, kwargs.pop(name, defaults[name]))
        kwargs.setdefault("architectures", [ARCHITECTURE])
        kwargs.setdefault("tie_word_embeddings", False)
        super().__init__(**kwargs)

    def to_native(self) -> LimiteConfig:
        values = {name: getattr(self, name) for name in _FIELDS}
        for name in ("global_layers", "ve_layers"):                 # JSON turns tuples into lists
            values[name] = tuple(values[name])
        return LimiteConfig(**values)

    @classmethod
    def from_native(cls, config: LimiteConfig) -> "LimiteHFConfig":
        return cls(**asdict(config))


class LimiteForCausalLM(PreTrainedModel):
    config_class = LimiteHFConfig
    base_model_prefix = "model"
    _no_split_modules = ["LimiteBlock"]

    def __init__(self, config: LimiteHFConfig):
        super().__init__(config)
        self.model = LimiteLM(config.to_native())
        self.post_init()

    def _init_weights(self, module):                                 # weights come from the checkpoint or init_weights()
        return

    def get_input_embeddings(self):
        return self.model.embed

    def get_output_embeddings(self):
        return self.model.lm_head

    def forward(self, input_ids: torch.Tensor, labels: torch.Tensor | None = None, **_unused) -> CausalLMOutput:
        logits = self.model(input_ids)
        loss = None
        if labels is not None:                                       # HF convention: labels are the inputs, shifted here
            shifted = torch.nn.functional.pad(labels[:, 1:], (0, 1), value=-100)
            loss = torch.nn.functional.cross_entropy(logits.flatten(0, 1), shifted.flatten(), ignore_index=-100)
        return CausalLMOutput(loss=loss, logits=logits)


def native_state(model: LimiteLM) -> dict[str, torch.Tensor]:
    """State dict under the names ``from_pretrained`` expects (``model.`` prefix)."""
    return {f"model.{k}": v for k, v in model.state_dict().items()}


def export_limite(out_dir, model: LimiteLM, *, lineage: dict | None = None) -> dict:
    from ..ckpt.formats import export_hf

    return export_hf(out_dir, native_state(model), LimiteHFConfig.from_native(model.config).to_dict(), lineage=lineage)


def register() -> None:
    AutoConfig.register(MODEL_TYPE, LimiteHFConfig, exist_ok=True)
    AutoModelForCausalLM.register(LimiteHFConfig, LimiteForCausalLM, exist_ok=True)
    try:
        from vllm import ModelRegistry
    except Exception:                                                # vLLM absent or unusable here: the HF side suffices
        return
    if ARCHITECTURE not in ModelRegistry.get_supported_archs():
        ModelRegistry.register_model(ARCHITECTURE, "archlab_b200.serve.hf_limite:LimiteForCausalLM")


register()
