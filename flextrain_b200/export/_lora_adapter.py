"""PEFT-format LoRA adapter export (flextrain/export/_lora_adapter.py:198): ``adapter_config.json`` +
``adapter_model.safetensors`` with ``base_model.model.<module>.lora_A/B.weight``.  Adapter tensors are already
in PEFT orientation (``A (r, in)``, ``B (out, r)``)."""
from __future__ import annotations

import json
import os

import torch

_MODULE = {"w_q": "self_attn.q_proj", "w_k": "self_attn.k_proj", "w_v": "self_attn.v_proj", "w_o": "self_attn.o_proj",
           "w_1": "mlp.gate_proj", "w_3": "mlp.up_proj", "w_2": "mlp.down_proj"}


def save_lora_adapter(am, out_dir: str, base_model_name_or_path: str = "") -> str:
    from safetensors.torch import save_file
    from ..io.hf_weights import gather_local_parts, is_export_writer
    lora = am.layers[0].cfg.lora
    if lora is None:
        raise ValueError("model was not built with LoRA")
    state = {}

    def whole(l, key, t):
        spec = am.layers[l].param_spec.get(key)
        if spec is not None and spec.is_local_part:            # tensor parallel: every rank takes part in the gather
            t = gather_local_parts(t.detach(), spec, am)
        return t.detach().to("cpu", torch.float32).contiguous()

    for l in range(len(am.layers)):
        p = am.buffers.host_params(l)
        for name, mod in _MODULE.items():
            if name + "_lora_a" in p:
                base = f"base_model.model.model.layers.{l}.{mod}"
                state[f"{base}.lora_A.weight"] = whole(l, name + "_lora_a", p[name + "_lora_a"])
                state[f"{base}.lora_B.weight"] = whole(l, name + "_lora_b", p[name + "_lora_b"])
    if not is_export_writer(am):
        return out_dir
    os.makedirs(out_dir, exist_ok=True)
    save_file(state, os.path.join(out_dir, "adapter_model.safetensors"), metadata={"format": "pt"})
    cfg = {"peft_type": "LORA", "task_type": "CAUSAL_LM", "r": lora.rank, "lora_alpha": lora.alpha,
           "lora_dropout": 0.0, "bias": "none", "fan_in_fan_out": False, "inference_mode": True,
           "target_modules": sorted({_MODULE[t].split(".")[-1] for t in lora.targets if t in _MODULE}),
           "base_model_name_or_path": base_model_name_or_path or (am.model_dir or "")}
    with open(os.path.join(out_dir, "adapter_config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    return out_dir
