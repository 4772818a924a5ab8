"""RoPE configuration: inverse-frequency builders and MRoPE sections.

Scaling types handled (flextrain/nn/blocks/rope.py:28-104, 141-205, 284-337): none/default,
``linear``, ``llama3`` band scaling, partial rotary (first ``rotary_dim`` channels),
``proportional`` (Gemma-4 style: angles over the full head, zero-angle tail) and interleaved
MRoPE with (t, h, w) sections.  Channel pairing is rotate-half ``(i, i + rot/2)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from ...ops import reference as ref


@dataclass
class RopeConfig:
    theta: float = 10000.0
    scaling: Optional[dict] = None
    partial_rotary_factor: float = 1.0
    mrope_sections: Optional[Tuple[int, int, int]] = None

    def rotary_dim(self, head_dim: int) -> int:
        r = int(head_dim * self.partial_rotary_factor)
        return r - (r % 2)

    def inv_freq(self, head_dim: int) -> torch.Tensor:
        kind = (self.scaling or {}).get("rope_type", (self.scaling or {}).get("type", "default"))
        if kind == "proportional":
            sc = dict(self.scaling)
            sc.setdefault("partial_rotary_factor", self.partial_rotary_factor)
            return ref.rope_inv_freq(head_dim, self.theta, scaling=sc)
        return ref.rope_inv_freq(head_dim, self.theta, rotary_dim=self.rotary_dim(head_dim), scaling=self.scaling)

    @staticmethod
    def from_hf(cfg: dict, head_dim: int) -> "RopeConfig":
        """Read ``rope_theta`` / ``rope_scaling`` / ``partial_rotary_factor`` / ``mrope_section`` from an HF config."""
        rs = cfg.get("rope_scaling") or cfg.get("rope_parameters") or None
        # the nested parameter set is what transformers >= 5 reads; top-level keys are the older spelling
        theta = float((rs or {}).get("rope_theta", cfg.get("rope_theta", 10000.0)))
        sections = None
        scaling = None
        if rs:
            if "mrope_section" in rs:
                sections = tuple(int(x) for x in rs["mrope_section"])
            kind = rs.get("rope_type", rs.get("type", "default"))
            if kind not in ("default", "mrope", None):
                scaling = dict(rs)
        prf = float((rs or {}).get("partial_rotary_factor", cfg.get("partial_rotary_factor", 1.0)))
        return RopeConfig(theta=theta, scaling=scaling, partial_rotary_factor=prf, mrope_sections=sections)
