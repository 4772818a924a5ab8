"""Architecture registry (flextrain/io/arch/__init__.py:43-56).

Each module exposes ``ARCH_SPEC`` (checkpoint name map), ``config_from_hf(hf_config)``,
``config_from_dims(dims, hyperparams)``, ``default_hyperparams()``, ``to_hf_config(model_config)``.
"""
from __future__ import annotations

import importlib
from typing import Optional

ARCH_MODULES = {
    "llama": "llama", "mistral": "mistral", "qwen2": "qwen2", "qwen3": "qwen3", "qwen3_moe": "qwen3_moe",
    "olmoe": "olmoe", "gemma2": "gemma2", "gemma3": "gemma3", "gemma3_text": "gemma3", "gemma4": "gemma4",
    "qwen3_5": "qwen3_5", "qwen3_5_moe": "qwen3_5_moe", "qwen3_next": "qwen3_next",
}

_HF_ARCHITECTURES = {
    "LlamaForCausalLM": "llama", "MistralForCausalLM": "mistral", "Qwen2ForCausalLM": "qwen2",
    "Qwen3ForCausalLM": "qwen3", "Qwen3MoeForCausalLM": "qwen3_moe", "OlmoeForCausalLM": "olmoe",
    "Gemma2ForCausalLM": "gemma2", "Gemma3ForCausalLM": "gemma3", "Gemma3ForConditionalGeneration": "gemma3",
    "Gemma4ForCausalLM": "gemma4", "Gemma4ForConditionalGeneration": "gemma4",
    "Qwen3_5ForCausalLM": "qwen3_5", "Qwen3_5ForConditionalGeneration": "qwen3_5",
    "Qwen3_5MoeForCausalLM": "qwen3_5_moe", "Qwen3_5MoeForConditionalGeneration": "qwen3_5_moe",
    "Qwen3NextForCausalLM": "qwen3_next",
}


def register_arch(key: str, module_name: str, hf_architectures=()) -> None:
    ARCH_MODULES[key] = module_name
    for a in hf_architectures:
        _HF_ARCHITECTURES[a] = key


def select_arch_module(arch: str, model_type: Optional[str] = None):
    """Resolve an HF ``architectures`` entry, a ``model_type`` or a family key to its module."""
    key = _HF_ARCHITECTURES.get(arch, arch)
    if key not in ARCH_MODULES and model_type in ARCH_MODULES:
        key = model_type
    if key not in ARCH_MODULES:
        raise KeyError(f"unsupported architecture {arch!r} (model_type={model_type!r}); known: {sorted(ARCH_MODULES)}")
    name = ARCH_MODULES[key]
    return importlib.import_module(f"{__name__}.{name}" if "." not in name else name)


select_arch = select_arch_module
get_arch_module = select_arch_module          # the reference's name (flextrain/io/arch/__init__.py:57-70)


def expand_layer_pattern(pattern: str, n_layers: int) -> list:
    """``"3L1F"`` and the like -> one layer type per layer (see :func:`.common.expand_layer_pattern`)."""
    from .common import expand_layer_pattern as _expand
    return _expand(pattern, n_layers)
