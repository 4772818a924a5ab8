"""Gemma 4 text tower.  Supported subset: the Gemma-3 layer shape with proportional partial RoPE on global
layers.  Checkpoints whose global layers share K and V (``k_eq_v``) or use per-layer head dims are rejected
with a clear error: the reference's own backward for those paths is a stub
(flextrain/nn/blocks/attention_gemma4.py:722), so there is no training behaviour to match."""
from __future__ import annotations

from ...nn.blocks.rope import RopeConfig
from ..hf_weights import ArchSpec
from . import _maps as M
from . import gemma2 as _g
from . import gemma3 as _g3
from .common import ModelConfig

FAMILY = "gemma4"
default_hyperparams = _g3.default_hyperparams


def config_from_dims(dims, hyper):
    mc = _g3.config_from_dims(dims, hyper)
    mc.arch = FAMILY
    return mc


def config_from_hf(hf: dict) -> ModelConfig:
    txt = hf.get("text_config", hf)
    if txt.get("attention_k_eq_v") or txt.get("global_head_dim") not in (None, txt.get("head_dim")):
        raise NotImplementedError("Gemma-4 checkpoints with shared K/V or per-layer head dims are not trainable here")
    mc = _g3.config_from_hf(hf)
    mc.arch = FAMILY
    prf = float(txt.get("global_partial_rotary_factor", txt.get("partial_rotary_factor", 1.0)))
    if prf < 1.0:
        mc.rope = RopeConfig(theta=mc.rope.theta, scaling={"rope_type": "proportional", "partial_rotary_factor": prf},
                             partial_rotary_factor=1.0)
    return mc


def to_hf_config(mc: ModelConfig) -> dict:
    c = _g3.to_hf_config(mc)
    c.update({"architectures": ["Gemma4ForCausalLM"], "model_type": "gemma4_text"})
    return c


ARCH_SPEC = ArchSpec(FAMILY, M.embed_entries, M.head_entries, _g._layer,
                     ("Gemma4ForCausalLM", "Gemma4ForConditionalGeneration"))
