"""Merged export: fold ``W += scale * B @ A`` into the base weights in fp32 on the CPU, then write a full HF
directory (flextrain/export/_merged.py:63,133)."""
from __future__ import annotations

import torch


def merged_weight(params, name: str, am) -> torch.Tensor:
    lora = am.layers[0].cfg.lora
    w = params[name].detach().to("cpu", torch.float32)
    a = params[name + "_lora_a"].detach().to("cpu", torch.float32)
    b = params[name + "_lora_b"].detach().to("cpu", torch.float32)
    if w.dim() == 3:      # per-expert adapters: (E, out, r) @ (E, r, in)
        return (w + lora.scale * torch.bmm(b, a)).to(params[name].dtype)
    return (w + lora.scale * (b @ a)).to(params[name].dtype)


def merge_lora_into_base(am) -> None:
    """In-place merge on the engine's master weights; adapters are reset to the identity (B = 0)."""
    for l in range(len(am.layers)):
        p = am.buffers.host_params(l)
        for name in [n for n in list(p) if (n + "_lora_a") in p]:
            p[name].copy_(merged_weight(p, name, am).to(p[name].device))
            p[name + "_lora_b"].zero_()


def save_hf_merged(am, out_dir: str, **kw) -> str:
    from ._hf_full import save_hf_full
    return save_hf_full(am, out_dir, _merge_lora=True, **kw)
