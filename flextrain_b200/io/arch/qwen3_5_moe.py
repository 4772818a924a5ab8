"""Qwen3.5-MoE (e.g. 35B-A3B): the Qwen3.5 hybrid mixer with routed experts + gated shared expert."""
from __future__ import annotations

from ..hf_weights import ArchSpec
from . import _maps as M
from . import qwen3_next as _n
from .common import ModelConfig

FAMILY = "qwen3_5_moe"
default_hyperparams = _n.default_hyperparams


def config_from_dims(dims, hyper):
    mc = _n.config_from_dims(dims, hyper)
    mc.arch = FAMILY
    return mc


def config_from_hf(hf: dict) -> ModelConfig:
    return _n.hybrid_from_hf(hf, FAMILY)


def to_hf_config(mc: ModelConfig) -> dict:
    c = _n.to_hf_config(mc)
    c.update({"architectures": ["Qwen3_5MoeForCausalLM"], "model_type": "qwen3_5_moe_text"})
    return c


ARCH_SPEC = ArchSpec(FAMILY, M.embed_entries, M.head_entries, _n._layer,
                     ("Qwen3_5MoeForCausalLM", "Qwen3_5MoeForConditionalGeneration"))
