"""Qwen3.5 dense hybrid (Gated DeltaNet + gated attention, dense SwiGLU FFN, MRoPE-capable text tower)
(flextrain/nn/layers/qwen3_5.py)."""
from __future__ import annotations

from ..hf_weights import ArchSpec
from . import _maps as M
from . import qwen3_next as _n
from .common import ModelConfig

FAMILY = "qwen3_5"
default_hyperparams = _n.default_hyperparams


def config_from_dims(dims, hyper):
    mc = _n.config_from_dims(dims, hyper)
    mc.arch = FAMILY
    return mc


def config_from_hf(hf: dict) -> ModelConfig:
    return _n.hybrid_from_hf(hf, FAMILY)


def to_hf_config(mc: ModelConfig) -> dict:
    c = _n.to_hf_config(mc)
    c.update({"architectures": ["Qwen3_5ForCausalLM"], "model_type": "qwen3_5_text"})
    return c


ARCH_SPEC = ArchSpec(FAMILY, M.embed_entries, M.head_entries, _n._layer,
                     ("Qwen3_5ForCausalLM", "Qwen3_5ForConditionalGeneration"))
