"""Frozen Qwen3-VL / Qwen3.5 vision tower in plain PyTorch (flextrain/nn/encoders/qwen_vl_vit.py:1-50).

Structure (it follows the published architecture, checked against ``transformers``' ``Qwen3_5VisionModel``):

* patch embedding: a strided 3-D convolution over ``temporal_patch x patch x patch`` pixel blocks, i.e. a linear map
  (with bias) of the flattened block;
* a learned ``num_pos`` position table laid out on a square grid and bilinearly interpolated to each image's
  ``h x w`` patch grid;
* ``depth`` pre-LayerNorm blocks: full (non-causal) attention inside every frame with 2-D rotary embeddings (half of
  the rotary slots from the patch row, half from the column) and a two-layer MLP;
* a patch merger: LayerNorm, then every ``merge x merge`` block of neighbouring patches is concatenated and projected
  to the language model's width by a two-layer GELU MLP.

Patches arrive in merge-block-major order (the four patches of a block are consecutive), as the HuggingFace image
processors emit them, so the merger is a plain reshape.  The tower runs under ``torch.inference_mode`` once per
round and never trains in this phase; attention is PyTorch SDPA per frame (head dims such as 72 are outside the
tcgen05 attention kernel's 64 / 128)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


@dataclass
class ViTConfig:
    depth: int = 27
    hidden: int = 1152
    heads: int = 16
    mlp: int = 4304
    patch: int = 16
    temporal_patch: int = 2
    in_chans: int = 3
    merge: int = 2
    out_hidden: int = 2048
    num_pos: int = 2304
    act: str = "gelu_pytorch_tanh"
    eps: float = 1e-6
    rope_theta: float = 10000.0

    @staticmethod
    def from_hf(v: dict) -> "ViTConfig":
        return ViTConfig(depth=v.get("depth", 27), hidden=v.get("hidden_size", v.get("embed_dim", 1152)),
                         heads=v.get("num_heads", 16), mlp=v.get("intermediate_size", 4304),
                         patch=v.get("patch_size", 16), temporal_patch=v.get("temporal_patch_size", 2),
                         in_chans=v.get("in_channels", v.get("in_chans", 3)), merge=v.get("spatial_merge_size", 2),
                         out_hidden=v.get("out_hidden_size", v.get("hidden_size", 2048)),
                         num_pos=v.get("num_position_embeddings", 2304), act=v.get("hidden_act", "gelu_pytorch_tanh"))

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def patch_dim(self) -> int:
        return self.in_chans * self.temporal_patch * self.patch * self.patch


def _act(name: str, x: torch.Tensor) -> torch.Tensor:
    if name in ("gelu_pytorch_tanh", "gelu_tanh"):
        return F.gelu(x, approximate="tanh")
    if name == "gelu":
        return F.gelu(x)
    if name in ("silu", "swish"):
        return F.silu(x)
    if name == "quick_gelu":
        return x * torch.sigmoid(1.702 * x)
    raise ValueError(f"unsupported vision activation {name!r}")


class QwenVLViT:
    """Holds the tower's tensors in a flat ``{name: tensor}`` dict with the checkpoint's own names."""

    PREFIXES = ("model.visual.", "visual.", "model.language_model.visual.")

    def __init__(self, cfg: ViTConfig, device="cpu", dtype=torch.float32):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        self.w: Dict[str, torch.Tensor] = {}
        self.master: Optional[Dict[str, torch.Tensor]] = None      # fp32 leaves when the tower trains
        self._ckpt_shapes: Dict[str, tuple] = {}                   # shapes as the checkpoint stores them (conv kernels)
        self.loaded_prefix = self.PREFIXES[0]                      # where the checkpoint keeps the tower

    # ------------------------------------------------------------------ parameters
    def param_shapes(self) -> Dict[str, tuple]:
        c = self.cfg
        s = {"patch_embed.proj.weight": (c.hidden, c.patch_dim), "patch_embed.proj.bias": (c.hidden,),
             "pos_embed.weight": (c.num_pos, c.hidden)}
        for i in range(c.depth):
            p = f"blocks.{i}."
            s.update({p + "norm1.weight": (c.hidden,), p + "norm1.bias": (c.hidden,),
                      p + "norm2.weight": (c.hidden,), p + "norm2.bias": (c.hidden,),
                      p + "attn.qkv.weight": (3 * c.hidden, c.hidden), p + "attn.qkv.bias": (3 * c.hidden,),
                      p + "attn.proj.weight": (c.hidden, c.hidden), p + "attn.proj.bias": (c.hidden,),
                      p + "mlp.linear_fc1.weight": (c.mlp, c.hidden), p + "mlp.linear_fc1.bias": (c.mlp,),
                      p + "mlp.linear_fc2.weight": (c.hidden, c.mlp), p + "mlp.linear_fc2.bias": (c.hidden,)})
        m = c.hidden * c.merge * c.merge
        s.update({"merger.norm.weight": (c.hidden,), "merger.norm.bias": (c.hidden,),
                  "merger.linear_fc1.weight": (m, m), "merger.linear_fc1.bias": (m,),
                  "merger.linear_fc2.weight": (c.out_hidden, m), "merger.linear_fc2.bias": (c.out_hidden,)})
        return s

    def num_params(self) -> int:
        n = 0
        for shp in self.param_shapes().values():
            k = 1
            for d in shp:
                k *= d
            n += k
        return n

    def init_random(self, seed: int = 0, std: float = 0.02) -> None:
        g = torch.Generator().manual_seed(seed)
        for n, shp in self.param_shapes().items():
            if n.endswith("bias"):
                t = torch.zeros(shp)
            elif "norm" in n:
                t = torch.ones(shp)
            else:
                t = torch.randn(shp, generator=g) * std
            self.w[n] = t.to(self.device, self.dtype)

    def load_state(self, state: Dict[str, torch.Tensor]) -> None:
        """``state`` uses the tower's own names (no prefix); convolution kernels are flattened to matrices."""
        for n, shp in self.param_shapes().items():
            t = state[n]
            self._ckpt_shapes[n] = tuple(t.shape)
            if t.dim() > 2:
                t = t.reshape(t.shape[0], -1)
            if tuple(t.shape) != tuple(shp):
                raise ValueError(f"vision tower tensor {n}: checkpoint {tuple(t.shape)} != expected {tuple(shp)}")
            self.w[n] = t.detach().to(self.device, self.dtype).contiguous()

    def load(self, reader, prefix: str = None) -> None:
        """Read the tower from a safetensors directory reader; the prefix is searched when not given."""
        prefixes = (prefix,) if prefix else self.PREFIXES
        probe = "patch_embed.proj.weight"
        for pre in prefixes:
            if reader.has(pre + probe):
                self.load_state({n: reader.get(pre + n) for n in self.param_shapes()})
                self.loaded_prefix = pre
                return
        raise KeyError(f"no vision tower found under any of {prefixes}")

    # ----------------------------------------------------------------- position data
    def _block_order(self, h: int, w: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Row / column of every patch of an ``h x w`` grid in merge-block-major order."""
        m = self.cfg.merge
        rows = torch.arange(h, device=self.device).view(h // m, 1, m, 1).expand(h // m, w // m, m, m).reshape(-1)
        cols = torch.arange(w, device=self.device).view(1, w // m, 1, m).expand(h // m, w // m, m, m).reshape(-1)
        return rows, cols

    def _rotary_angles(self, t: int, h: int, w: int) -> torch.Tensor:
        """``(t*h*w, head_dim/2)``: the first half of the slots rotates with the patch row, the second with the column."""
        quarter = self.cfg.head_dim // 2
        inv = 1.0 / (self.cfg.rope_theta ** (torch.arange(0, quarter, 2, dtype=torch.float32, device=self.device) / quarter))
        rows, cols = self._block_order(h, w)
        ang = torch.cat([rows.to(torch.float32)[:, None] * inv, cols.to(torch.float32)[:, None] * inv], -1)
        return ang.repeat(t, 1)

    def _pos_embed(self, t: int, h: int, w: int, table: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Bilinear interpolation of the square position table to ``h x w``, in merge-block-major order."""
        table = self.w["pos_embed.weight"] if table is None else table
        side = int(round(self.cfg.num_pos ** 0.5))
        hi = torch.linspace(0, side - 1, h, device=self.device)
        wi = torch.linspace(0, side - 1, w, device=self.device)
        h0, w0 = hi.int(), wi.int()
        h1, w1 = (h0 + 1).clamp(max=side - 1), (w0 + 1).clamp(max=side - 1)
        dh, dw = (hi - h0).to(table.dtype), (wi - w0).to(table.dtype)

        def corner(hh, ww, wh, wwt):
            idx = (hh.long() * side)[:, None] + ww.long()[None, :]
            return table[idx.reshape(-1)] * (wh[:, None] * wwt[None, :]).reshape(-1, 1)

        grid = corner(h0, w0, 1 - dh, 1 - dw) + corner(h0, w1, 1 - dh, dw) + corner(h1, w0, dh, 1 - dw) \
            + corner(h1, w1, dh, dw)                                        # (h*w, hidden), row-major
        rows, cols = self._block_order(h, w)
        return grid[rows * w + cols].repeat(t, 1)

    @staticmethod
    def _rotate(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        d = x.shape[-1] // 2
        xf = x.float()
        rot = torch.cat([-xf[..., d:], xf[..., :d]], -1)
        return (xf * cos + rot * sin).to(x.dtype)

    # ----------------------------------------------------------------------- forward
    # ---------------------------------------------------------------------- training
    def enable_training(self) -> None:
        """Make the tower trainable: fp32 master copies become autograd leaves (their ``.grad`` accumulates over the
        rounds of a step); the compute-dtype copies in ``self.w`` are refreshed after every update."""
        self.master = {n: t.detach().to(torch.float32).clone().requires_grad_(True) for n, t in self.w.items()}

    @property
    def trainable(self) -> bool:
        return self.master is not None

    def param_spec(self):
        """The tower's tensors as a :class:`ParamSpec` (fp32 master and gradient), for the engine's optimizer."""
        from ...core.layer import ParamSpec, TensorSpec
        return ParamSpec([TensorSpec(n, tuple(t.shape), self.dtype, master_dtype=torch.float32, grad_dtype=torch.float32,
                                     opt_state_dtype=torch.float32) for n, t in self.w.items()])

    def sync_compute(self) -> None:
        for n, m in (self.master or {}).items():
            self.w[n] = m.detach().to(self.dtype)

    def encode_train(self, pixel_values: torch.Tensor, grid_thw: Sequence[Sequence[int]]) -> torch.Tensor:
        """Like :meth:`encode`, with the autograd graph kept: ``rows.backward(d_rows)`` adds into ``master[n].grad``."""
        if self.master is None:
            raise RuntimeError("enable_training() first")
        with torch.enable_grad():
            return self._forward({n: m.to(self.dtype) for n, m in self.master.items()}, pixel_values, grid_thw, False)

    def export_state(self) -> Dict[str, torch.Tensor]:
        """Current weights under the tower's own names, in the checkpoint's shapes (conv kernels un-flattened)."""
        src = self.master if self.master is not None else self.w
        return {n: t.detach().to("cpu", self.w[n].dtype).reshape(self._ckpt_shapes.get(n, tuple(t.shape))).contiguous()
                for n, t in src.items()}

    @torch.inference_mode()
    def encode(self, pixel_values: torch.Tensor, grid_thw: Sequence[Sequence[int]], return_hidden: bool = False):
        """``pixel_values (n_patches, C*tp*p*p)`` of all images, ``grid_thw`` = ``(t, h, w)`` per image (in patches).
        Returns the merged rows ``(n_patches / merge**2, out_hidden)`` in image order."""
        return self._forward(self.w, pixel_values, grid_thw, return_hidden)

    def _forward(self, W: Dict[str, torch.Tensor], pixel_values: torch.Tensor, grid_thw, return_hidden: bool):
        c = self.cfg
        grids = [tuple(int(v) for v in g) for g in (grid_thw.tolist() if torch.is_tensor(grid_thw) else grid_thw)]
        n_expected = sum(t * h * w for t, h, w in grids)
        if pixel_values.shape[0] != n_expected or pixel_values.shape[1] != c.patch_dim:
            raise ValueError(f"pixel_values {tuple(pixel_values.shape)} does not match grids {grids} "
                             f"(expected ({n_expected}, {c.patch_dim}))")
        x = F.linear(pixel_values.to(self.device, self.dtype), W["patch_embed.proj.weight"], W["patch_embed.proj.bias"])
        x = x + torch.cat([self._pos_embed(t, h, w, W["pos_embed.weight"]) for t, h, w in grids], 0)
        ang = torch.cat([self._rotary_angles(t, h, w) for t, h, w in grids], 0)
        ang = torch.cat([ang, ang], -1)
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        frames: List[int] = []                               # attention never crosses a frame
        for t, h, w in grids:
            frames += [h * w] * t
        n, hd = x.shape[0], c.head_dim
        for i in range(c.depth):
            p = f"blocks.{i}."
            hn = F.layer_norm(x, (c.hidden,), W[p + "norm1.weight"], W[p + "norm1.bias"], c.eps)
            qkv = F.linear(hn, W[p + "attn.qkv.weight"], W[p + "attn.qkv.bias"]).view(n, 3, c.heads, hd)
            q, k, v = self._rotate(qkv[:, 0], cos, sin), self._rotate(qkv[:, 1], cos, sin), qkv[:, 2]
            outs, off = [], 0
            for L in frames:
                sl = slice(off, off + L)
                o = F.scaled_dot_product_attention(q[sl].transpose(0, 1)[None], k[sl].transpose(0, 1)[None],
                                                   v[sl].transpose(0, 1)[None])
                outs.append(o[0].transpose(0, 1).reshape(L, c.hidden))
                off += L
            x = x + F.linear(torch.cat(outs, 0), W[p + "attn.proj.weight"], W[p + "attn.proj.bias"])
            hn = F.layer_norm(x, (c.hidden,), W[p + "norm2.weight"], W[p + "norm2.bias"], c.eps)
            hn = _act(c.act, F.linear(hn, W[p + "mlp.linear_fc1.weight"], W[p + "mlp.linear_fc1.bias"]))
            x = x + F.linear(hn, W[p + "mlp.linear_fc2.weight"], W[p + "mlp.linear_fc2.bias"])
        y = F.layer_norm(x, (c.hidden,), W["merger.norm.weight"], W["merger.norm.bias"], c.eps)
        y = y.view(-1, c.hidden * c.merge * c.merge)         # block-major order: a block's patches are consecutive
        y = F.gelu(F.linear(y, W["merger.linear_fc1.weight"], W["merger.linear_fc1.bias"]))
        y = F.linear(y, W["merger.linear_fc2.weight"], W["merger.linear_fc2.bias"])
        return (y, x) if return_hidden else y

    def rows_per_image(self, grid_thw: Sequence[Sequence[int]]) -> List[int]:
        m2 = self.cfg.merge ** 2
        return [int(t) * int(h) * int(w) // m2 for t, h, w in grid_thw]
