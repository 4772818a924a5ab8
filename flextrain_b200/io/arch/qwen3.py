"""Qwen3 dense: per-head QK RMSNorm, no biases, optional sliding-window layers
(flextrain/nn/layers/qwen3.py)."""
from __future__ import annotations

from ..hf_weights import ArchSpec
from . import _maps as M
from . import llama as _l
from .common import ModelConfig, config_from_dims as _cfd

FAMILY = "qwen3"


def default_hyperparams() -> dict:
    return {"rope_theta": 1000000.0, "norm_eps": 1e-6, "qk_norm": "head"}


def config_from_dims(dims, hyper):
    return _cfd(dims, FAMILY, hyper)


def config_from_hf(hf: dict) -> ModelConfig:
    mc = _l.config_from_hf(hf)
    mc.arch, mc.qk_norm = FAMILY, "head"
    lt = hf.get("layer_types")
    if lt and hf.get("use_sliding_window", False):
        mc.layer_types = ["sliding" if t == "sliding_attention" else "full" for t in lt]
        mc.sliding_window = int(hf.get("sliding_window") or 0)
    return mc


def to_hf_config(mc: ModelConfig) -> dict:
    c = _l.to_hf_config(mc)
    c.update({"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3"})
    return c


ARCH_SPEC = ArchSpec(FAMILY, M.embed_entries, M.head_entries, _l._layer, ("Qwen3ForCausalLM",))
