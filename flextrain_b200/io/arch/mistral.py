"""Mistral: Llama-shaped with an optional sliding window on every layer (flextrain/nn/layers/mistral.py)."""
from __future__ import annotations

from ..hf_weights import ArchSpec
from . import _maps as M
from . import llama as _l
from .common import ModelConfig, config_from_dims as _cfd

FAMILY = "mistral"


def default_hyperparams() -> dict:
    return {"rope_theta": 1000000.0, "norm_eps": 1e-5}


def config_from_dims(dims, hyper):
    return _cfd(dims, FAMILY, hyper)


def config_from_hf(hf: dict) -> ModelConfig:
    mc = _l.config_from_hf(hf)
    mc.arch = FAMILY
    sw = hf.get("sliding_window")
    if sw:
        mc.sliding_window = int(sw)
        mc.layer_types = ["sliding"] * mc.n_layers
    return mc


def to_hf_config(mc: ModelConfig) -> dict:
    c = _l.to_hf_config(mc)
    c.update({"architectures": ["MistralForCausalLM"], "model_type": "mistral",
              "sliding_window": mc.sliding_window or None})
    return c


ARCH_SPEC = ArchSpec(FAMILY, M.embed_entries, M.head_entries, _l._layer, ("MistralForCausalLM",))
