"""Gemma 4 text tower (dense layers).  On top of the Gemma-3 layer shape (sandwich norms, per-head QK-norm, sliding /
global layers with their own RoPE bases, tanh-GeGLU, ``sqrt(d)`` embedding scale, tied head) Gemma 4 changes:

* norm weights are stored as the gain itself (Gemma 2 / 3 store gain - 1);
* V gets a per-head RMSNorm without a learned gain, and the attention logits are not scaled (scale 1.0);
* global layers use *proportional* partial RoPE: the first ``partial_rotary_factor`` of the frequency pairs rotate
  with exponents taken over the whole head dim, the rest stay unrotated;
* every layer's output is multiplied by a stored, untrained ``layer_scalar``.

Checkpoints whose global layers share K and V (``attention_k_eq_v``), use a different global head dim, share KV across
layers, carry per-layer input embeddings or the MoE branch are rejected with a clear error: the reference's own
backward for this family is a stub (flextrain/nn/blocks/attention_gemma4.py:722, flextrain/nn/layers/gemma4.py), so
there is no training behaviour to match beyond the dense path, which is checked against ``transformers``."""
from __future__ import annotations

from typing import List

from ...nn.blocks.rope import RopeConfig
from ..hf_weights import ArchSpec, WeightMapEntry as E
from . import _maps as M
from . import gemma2 as _g
from . import gemma3 as _g3
from .common import ModelConfig

FAMILY = "gemma4"


def default_hyperparams() -> dict:
    return {**_g3.default_hyperparams(), "v_norm": True, "layer_scalar": True, "attn_scale": 1.0,
            "rope_scaling": {"rope_type": "proportional", "partial_rotary_factor": 0.25}}


def config_from_dims(dims, hyper):
    mc = _g3.config_from_dims(dims, {**default_hyperparams(), **hyper})
    mc.arch = FAMILY
    mc.norm_plus_one = False
    return mc


_UNSUPPORTED = (("attention_k_eq_v", "global layers that share K and V"),
                ("hidden_size_per_layer_input", "per-layer input embeddings"),
                ("enable_moe_block", "the MoE branch"),
                ("num_kv_shared_layers", "KV sharing across layers"),
                ("use_double_wide_mlp", "double-wide MLPs"))


def _rope_of(params: dict, default_theta: float) -> RopeConfig:
    kind = params.get("rope_type", "default")
    theta = float(params.get("rope_theta", default_theta))
    if kind == "proportional":
        prf = float(params.get("partial_rotary_factor", 1.0))
        return RopeConfig(theta=theta, scaling={"rope_type": "proportional", "partial_rotary_factor": prf})
    return RopeConfig(theta=theta, scaling=None if kind == "default" else dict(params))


def config_from_hf(hf: dict) -> ModelConfig:
    txt = hf.get("text_config", hf)
    for key, what in _UNSUPPORTED:
        if txt.get(key):
            raise NotImplementedError(f"Gemma-4 checkpoints with {what} ({key}={txt[key]!r}) are not trainable here")
    if txt.get("global_head_dim") not in (None, txt.get("head_dim")):
        raise NotImplementedError("Gemma-4 checkpoints with a separate global head dim are not trainable here")
    mc = _g3.config_from_hf(hf)
    mc.arch = FAMILY
    mc.norm_plus_one = False
    mc.attn_scale, mc.v_norm, mc.layer_scalar = 1.0, True, True
    mc.final_softcap = float(txt.get("final_logit_softcapping") or 0.0)
    rp = txt.get("rope_parameters") or {}
    if "full_attention" in rp or "sliding_attention" in rp:
        mc.rope = _rope_of(rp.get("full_attention", {}), 1000000.0)
        mc.rope_local = _rope_of(rp.get("sliding_attention", {}), 10000.0)
    else:
        prf = float(txt.get("global_partial_rotary_factor", txt.get("partial_rotary_factor", 1.0)))
        if prf < 1.0:
            mc.rope = RopeConfig(theta=mc.rope.theta, scaling={"rope_type": "proportional",
                                                               "partial_rotary_factor": prf})
    return mc


def to_hf_config(mc: ModelConfig) -> dict:
    c = _g3.to_hf_config(mc)
    for k in ("rope_theta", "rope_local_base_freq", "rope_scaling", "query_pre_attn_scalar"):
        c.pop(k, None)

    def params(r: RopeConfig) -> dict:
        if r.scaling and r.scaling.get("rope_type") == "proportional":
            return {"rope_type": "proportional", "rope_theta": r.theta,
                    "partial_rotary_factor": r.scaling.get("partial_rotary_factor", 1.0)}
        return {"rope_type": "default", "rope_theta": r.theta}

    c.update({"architectures": ["Gemma4ForCausalLM"], "model_type": "gemma4_text", "global_head_dim": mc.head_dim,
              "hidden_size_per_layer_input": 0, "final_logit_softcapping": mc.final_softcap or None,
              "rope_parameters": {"full_attention": params(mc.rope),
                                  "sliding_attention": params(mc.rope_local or RopeConfig(theta=10000.0))}})
    return c


def _layer(i: int, mc: ModelConfig) -> List:
    return _g._layer(i, mc) + [E("w_layer_scalar", [f"model.layers.{i}.layer_scalar"], optional=True)]


ARCH_SPEC = ArchSpec(FAMILY, M.embed_entries, M.head_entries, _layer,
                     ("Gemma4ForCausalLM", "Gemma4ForConditionalGeneration"))
