"""OLMoE-1B-7B: full-row QK RMSNorm, 64 routed experts (flextrain/nn/layers/olmoe.py)."""
from __future__ import annotations

from ..hf_weights import ArchSpec
from . import _maps as M
from . import llama as _l
from .common import ModelConfig, config_from_dims as _cfd

FAMILY = "olmoe"


def default_hyperparams() -> dict:
    return {"rope_theta": 10000.0, "norm_eps": 1e-5, "qk_norm": "row", "routing": "softmax_then_topk"}


def config_from_dims(dims, hyper):
    return _cfd(dims, FAMILY, hyper)


def config_from_hf(hf: dict) -> ModelConfig:
    mc = _l.config_from_hf(hf)
    mc.arch, mc.qk_norm = FAMILY, "row"
    mc.num_experts, mc.top_k = int(hf.get("num_experts", hf.get("num_local_experts"))), int(hf["num_experts_per_tok"])
    mc.expert_dim = int(hf["intermediate_size"])
    mc.routing = "topk_then_softmax" if hf.get("norm_topk_prob", False) else "softmax_then_topk"
    mc.aux_loss_alpha = float(hf.get("router_aux_loss_coef", 0.0)) if hf.get("output_router_logits") else 0.0
    return mc


def to_hf_config(mc: ModelConfig) -> dict:
    c = _l.to_hf_config(mc)
    c.update({"architectures": ["OlmoeForCausalLM"], "model_type": "olmoe", "num_experts": mc.num_experts,
              "num_experts_per_tok": mc.top_k, "intermediate_size": mc.expert_dim,
              "norm_topk_prob": mc.routing == "topk_then_softmax"})
    return c


ARCH_SPEC = ArchSpec(FAMILY, M.embed_entries, M.head_entries, _l._layer, ("OlmoeForCausalLM",))
