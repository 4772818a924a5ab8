"""Adding a model family from outside the package: Phi-3 (the reference's docs/extending/tutorial_phi3.md).

Phi-3 is a Llama-shaped decoder whose checkpoint fuses the attention projections into ``self_attn.qkv_proj``
(rows ``[q ‖ k ‖ v]``) and the MLP's gate / up projections into ``mlp.gate_up_proj`` (rows ``[gate ‖ up]``).  A family
needs exactly what this file has:

* ``config_from_hf`` / ``config_from_dims`` / ``default_hyperparams`` / ``to_hf_config``: the translation between an
  HF ``config.json`` (or a dims dict) and the engine's :class:`ModelConfig`;
* ``ARCH_SPEC``: the map between checkpoint tensors and engine tensors.  Loading a slice of a fused tensor is a
  ``combine`` callable on the entry; writing the fused tensor back is the spec's ``export_hook``;
* one ``register_arch`` call.  No layer code: the config-driven decoder layer already covers the architecture.

    import examples.extending_phi3          # registers "phi3" / Phi3ForCausalLM
    am = flextrain_b200.from_pretrained("/path/to/Phi-3-mini-4k-instruct", ...)

``tests/test_extending_cpu.py`` checks the result against ``transformers``' Phi-3 (loss, gradients, export)."""
from __future__ import annotations

from typing import Dict, List

import torch

from flextrain_b200.io.arch import _maps as M
from flextrain_b200.io.arch import llama as _llama
from flextrain_b200.io.arch import register_arch
from flextrain_b200.io.arch.common import ModelConfig, config_from_dims as _cfd
from flextrain_b200.io.hf_weights import ArchSpec, WeightMapEntry as E

FAMILY = "phi3"


def default_hyperparams() -> dict:
    return {"rope_theta": 10000.0, "norm_eps": 1e-5}


def config_from_dims(dims: dict, hyper: dict) -> ModelConfig:
    return _cfd(dims, FAMILY, hyper)


def config_from_hf(hf: dict) -> ModelConfig:
    scaling = hf.get("rope_scaling") or (hf.get("rope_parameters") or {})
    if scaling.get("rope_type", scaling.get("type", "default")) not in ("default", None):
        raise NotImplementedError("Phi-3 long-context checkpoints (longrope scaling) are not covered by this example")
    if float(hf.get("partial_rotary_factor", (hf.get("rope_parameters") or {}).get("partial_rotary_factor", 1.0))) != 1.0:
        raise NotImplementedError("partial rotary Phi variants are not covered by this example")
    mc = _llama.config_from_hf(hf)
    mc.arch = FAMILY
    if hf.get("sliding_window") and hf["sliding_window"] < hf.get("max_position_embeddings", 1 << 30):
        mc.sliding_window = int(hf["sliding_window"])
        mc.layer_types = ["sliding"] * mc.n_layers
    return mc


def to_hf_config(mc: ModelConfig) -> dict:
    c = _llama.to_hf_config(mc)
    c.update({"architectures": ["Phi3ForCausalLM"], "model_type": "phi3", "max_position_embeddings": 4096,
              "original_max_position_embeddings": 4096, "sliding_window": mc.sliding_window or None,
              "pad_token_id": None})
    c.pop("head_dim", None); c.pop("attention_bias", None); c.pop("rope_scaling", None)
    return c


def _layer(i: int, mc: ModelConfig) -> List[E]:
    p = f"model.layers.{i}."
    q, kv, f = mc.n_heads * mc.head_dim, mc.n_kv_heads * mc.head_dim, mc.ffn_dim

    def rows(name: str, fused: str, a: int, b: int) -> E:
        # load: the entry's alternate is the checkpoint's fused tensor, of which it takes rows [a, b);
        # export: it is written under a per-tensor key that export_hook (below) fuses again
        return E(name, [p + "__" + name], alternates=[[p + fused]], combine=lambda ts: ts[0][a:b])

    fused = [rows("w_q", "self_attn.qkv_proj.weight", 0, q), rows("w_k", "self_attn.qkv_proj.weight", q, q + kv),
             rows("w_v", "self_attn.qkv_proj.weight", q + kv, q + 2 * kv),
             rows("w_1", "mlp.gate_up_proj.weight", 0, f), rows("w_3", "mlp.gate_up_proj.weight", f, 2 * f)]
    plain = [e for e in M.norm_entries(i, mc) + M.attn_entries(i, mc) + M.dense_ffn_entries(i, mc)
             if e.name in ("w_attn_norm", "w_ffn_norm", "w_o", "w_2")]
    return plain + fused


def _export_hook(state: Dict[str, torch.Tensor], mc: ModelConfig) -> Dict[str, torch.Tensor]:
    for i in range(mc.n_layers):
        p = f"model.layers.{i}."
        state[p + "self_attn.qkv_proj.weight"] = torch.cat([state.pop(p + "__w_q"), state.pop(p + "__w_k"),
                                                            state.pop(p + "__w_v")], 0)
        state[p + "mlp.gate_up_proj.weight"] = torch.cat([state.pop(p + "__w_1"), state.pop(p + "__w_3")], 0)
    return state


ARCH_SPEC = ArchSpec(FAMILY, M.embed_entries, M.head_entries, _layer, ("Phi3ForCausalLM",), export_hook=_export_hook)

register_arch(FAMILY, __name__, ("Phi3ForCausalLM",))
