"""Qwen2 / Qwen2.5: Llama-shaped with Q/K/V biases (flextrain/nn/layers/qwen2.py)."""
from __future__ import annotations

from ..hf_weights import ArchSpec
from . import _maps as M
from . import llama as _l
from .common import ModelConfig, config_from_dims as _cfd

FAMILY = "qwen2"


def default_hyperparams() -> dict:
    return {"rope_theta": 1000000.0, "norm_eps": 1e-6, "qkv_bias": True}


def config_from_dims(dims, hyper):
    return _cfd(dims, FAMILY, hyper)


def config_from_hf(hf: dict) -> ModelConfig:
    mc = _l.config_from_hf(hf)
    mc.arch, mc.qkv_bias = FAMILY, True
    return mc


def to_hf_config(mc: ModelConfig) -> dict:
    c = _l.to_hf_config(mc)
    c.update({"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2"})
    c.pop("attention_bias", None)
    return c


ARCH_SPEC = ArchSpec(FAMILY, M.embed_entries, M.head_entries, _l._layer, ("Qwen2ForCausalLM",))
