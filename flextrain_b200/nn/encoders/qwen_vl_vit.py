"""Frozen Qwen-VL vision tower in plain PyTorch (flextrain/nn/encoders/qwen_vl_vit.py:1-50).

Patch embedding (a linear map of flattened ``temporal x patch x patch`` pixels), ``depth`` pre-norm transformer
blocks with 2-D rotary position embeddings over the (h, w) patch grid and full attention per image, and a patch
merger that concatenates ``merge x merge`` neighbouring patches and projects them to the language model width.
Run under ``torch.inference_mode`` once per round; it never trains in this phase."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch
import torch.nn.functional as F


@dataclass
class ViTConfig:
    depth: int = 24
    hidden: int = 1024
    heads: int = 16
    mlp: int = 4096
    patch: int = 14
    temporal_patch: int = 2
    in_chans: int = 3
    merge: int = 2
    out_hidden: int = 2048
    eps: float = 1e-6

    @staticmethod
    def from_hf(v: dict) -> "ViTConfig":
        return ViTConfig(depth=v.get("depth", 24), hidden=v.get("hidden_size", v.get("embed_dim", 1024)),
                         heads=v.get("num_heads", 16), mlp=v.get("intermediate_size", 4096),
                         patch=v.get("patch_size", 14), temporal_patch=v.get("temporal_patch_size", 2),
                         in_chans=v.get("in_channels", v.get("in_chans", 3)), merge=v.get("spatial_merge_size", 2),
                         out_hidden=v.get("out_hidden_size", v.get("hidden_size", 2048)))


class QwenVLViT:
    def __init__(self, cfg: ViTConfig, device="cpu", dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w: Dict[str, torch.Tensor] = {}

    def param_shapes(self) -> Dict[str, tuple]:
        c = self.cfg
        pd = c.in_chans * c.temporal_patch * c.patch * c.patch
        s = {"patch_embed.proj.weight": (c.hidden, pd)}
        for i in range(c.depth):
            p = f"blocks.{i}."
            s.update({p + "norm1.weight": (c.hidden,), p + "norm2.weight": (c.hidden,),
                      p + "attn.qkv.weight": (3 * c.hidden, c.hidden), p + "attn.qkv.bias": (3 * c.hidden,),
                      p + "attn.proj.weight": (c.hidden, c.hidden), p + "attn.proj.bias": (c.hidden,),
                      p + "mlp.gate_proj.weight": (c.mlp, c.hidden), p + "mlp.up_proj.weight": (c.mlp, c.hidden),
                      p + "mlp.down_proj.weight": (c.hidden, c.mlp)})
        m = c.hidden * c.merge * c.merge
        s.update({"merger.ln_q.weight": (c.hidden,), "merger.mlp.0.weight": (m, m), "merger.mlp.0.bias": (m,),
                  "merger.mlp.2.weight": (c.out_hidden, m), "merger.mlp.2.bias": (c.out_hidden,)})
        return s

    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        g = torch.Generator().manual_seed(seed)
        for n, shp in self.param_shapes().items():
            if "norm" in n or "ln_q" in n:
                t = torch.ones(shp)
            elif n.endswith("bias"):
                t = torch.zeros(shp)
            else:
                t = torch.randn(shp, generator=g) * std
            self.w[n] = t.to(self.device, self.dtype)

    def load(self, reader, prefix: str = "visual.") -> None:
        for n, shp in self.param_shapes().items():
            t = reader.get(prefix + n)
            if t.dim() > 2:
                t = t.reshape(t.shape[0], -1)
            self.w[n] = t.to(self.device, self.dtype)

    def _rot(self, h: int, w: int, dim: int) -> torch.Tensor:
        """2-D rotary angles ``(h*w, dim/2)``: first half of the frequency slots from the row, second from the column."""
        half = dim // 2
        inv = 1.0 / (10000.0 ** (torch.arange(0, half, 2, dtype=torch.float32, device=self.device) / half))
        ys = torch.arange(h, device=self.device, dtype=torch.float32).repeat_interleave(w)
        xs = torch.arange(w, device=self.device, dtype=torch.float32).repeat(h)
        return torch.cat([ys[:, None] * inv, xs[:, None] * inv], -1)

    @staticmethod
    def _apply_rot(x: torch.Tensor, ang: torch.Tensor) -> torch.Tensor:
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        d = x.shape[-1] // 2
        x1, x2 = x[..., :d], x[..., d:]
        return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)

    @torch.inference_mode()
    def encode(self, pixel_values: torch.Tensor, grid_thw) -> torch.Tensor:
        """``pixel_values (n_patches, C*tp*p*p)`` for all images; ``grid_thw`` list of (t, h, w). Returns merged rows."""
        c, W = self.cfg, self.w
        x = pixel_values.to(self.device, self.dtype) @ W["patch_embed.proj.weight"].t()
        outs, off = [], 0
        hd = c.hidden // c.heads
        for (t, h, w) in grid_thw:
            n = t * h * w
            xi = x[off:off + n]
            off += n
            ang = self._rot(h, w, hd).repeat(t, 1)
            for i in range(c.depth):
                p = f"blocks.{i}."
                hn = F.rms_norm(xi, (c.hidden,), W[p + "norm1.weight"], c.eps)
                qkv = hn @ W[p + "attn.qkv.weight"].t() + W[p + "attn.qkv.bias"]
                q, k, v = qkv.view(n, 3, c.heads, hd).unbind(1)
                q, k = self._apply_rot(q, ang), self._apply_rot(k, ang)
                a = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None],
                                                   v.transpose(0, 1)[None])[0].transpose(0, 1).reshape(n, c.hidden)
                xi = xi + a @ W[p + "attn.proj.weight"].t() + W[p + "attn.proj.bias"]
                hn = F.rms_norm(xi, (c.hidden,), W[p + "norm2.weight"], c.eps)
                g, u = hn @ W[p + "mlp.gate_proj.weight"].t(), hn @ W[p + "mlp.up_proj.weight"].t()
                xi = xi + (F.silu(g) * u) @ W[p + "mlp.down_proj.weight"].t()
            xi = F.rms_norm(xi, (c.hidden,), W["merger.ln_q.weight"], c.eps)
            m = c.merge
            xi = xi.view(t, h // m, m, w // m, m, c.hidden).permute(0, 1, 3, 2, 4, 5).reshape(-1, m * m * c.hidden)
            xi = F.gelu(xi @ W["merger.mlp.0.weight"].t() + W["merger.mlp.0.bias"])
            outs.append(xi @ W["merger.mlp.2.weight"].t() + W["merger.mlp.2.bias"])
        return torch.cat(outs, 0)
