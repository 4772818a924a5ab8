"""Qwen3-MoE (e.g. 30B-A3B): Qwen3 attention + routed SwiGLU experts, top-k then softmax
(flextrain/nn/layers/qwen3_moe.py)."""
from __future__ import annotations

from ..hf_weights import ArchSpec
from . import _maps as M
from . import llama as _l
from . import qwen3 as _q
from .common import ModelConfig, config_from_dims as _cfd

FAMILY = "qwen3_moe"


def default_hyperparams() -> dict:
    return {"rope_theta": 1000000.0, "norm_eps": 1e-6, "qk_norm": "head", "routing": "topk_then_softmax"}


def config_from_dims(dims, hyper):
    return _cfd(dims, FAMILY, hyper)


def config_from_hf(hf: dict) -> ModelConfig:
    mc = _q.config_from_hf(hf)
    mc.arch = FAMILY
    mc.num_experts, mc.top_k = int(hf.get("num_experts", hf.get("num_local_experts"))), int(hf["num_experts_per_tok"])
    mc.expert_dim = int(hf["moe_intermediate_size"])
    mc.routing = "topk_then_softmax" if hf.get("norm_topk_prob", True) else "softmax_then_topk"
    # the checkpoint's load-balance coefficient applies only when the config asks for router losses (HF semantics)
    mc.aux_loss_alpha = float(hf.get("router_aux_loss_coef", 0.0)) if hf.get("output_router_logits") else 0.0
    step = int(hf.get("decoder_sparse_step", 1) or 1)
    only_mlp = set(hf.get("mlp_only_layers", []) or [])
    mc.moe_layers = [((i + 1) % step == 0) and i not in only_mlp for i in range(mc.n_layers)]
    return mc


def to_hf_config(mc: ModelConfig) -> dict:
    c = _l.to_hf_config(mc)
    c.update({"architectures": ["Qwen3MoeForCausalLM"], "model_type": "qwen3_moe", "num_experts": mc.num_experts,
              "num_experts_per_tok": mc.top_k, "moe_intermediate_size": mc.expert_dim,
              "norm_topk_prob": mc.routing == "topk_then_softmax", "decoder_sparse_step": 1, "mlp_only_layers": []})
    return c


ARCH_SPEC = ArchSpec(FAMILY, M.embed_entries, M.head_entries, _l._layer, ("Qwen3MoeForCausalLM",))
