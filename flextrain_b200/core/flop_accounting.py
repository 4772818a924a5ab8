"""Authoritative FLOP accounting (flextrain/core/flop_accounting.py:111-460, train.py:110-151).

effective = forward + backward (2x forward for full fine-tuning, 1x for LoRA: no base weight gradients)
            + head (forward + 2 backward GEMMs) + optimizer;
hardware  = effective + recompute chosen by the save-level plan + 0.5 x attention forward (the flash
            backward re-scans the scores).
"""
from __future__ import annotations

from typing import Tuple


def fwd_flops(am, stats) -> float:
    return float(stats.fwd_flops)


def head_flops(am, tokens: int) -> float:
    return 2.0 * tokens * am.head.vocab_size * am.head.d_model


def bwd_flops(am, stats, mode: str = "full") -> float:
    return (2.0 if mode == "full" else 1.0) * float(stats.fwd_flops)


def opt_flops_per_step(am) -> float:
    """AdamW: ~12 FLOPs per trainable element. Muon: 5 Newton-Schulz iterations, each three matmuls on the
    (m x n, m <= n) matrix: ``2*m*m*n`` (X Xᵀ) + ``2*m*m*m`` (A²) + ``2*m*m*n`` (B X)."""
    from ..optim import HybridMuonAdamW, Muon, uses_muon
    opt = am.optimizer
    total = 0.0
    specs = [am.embed.param_spec, am.head.param_spec] + [l.param_spec for l in am.layers]
    for spec in specs:
        for t in spec.trainable():
            muon = isinstance(opt, Muon) or (isinstance(opt, HybridMuonAdamW) and uses_muon(t))
            if muon and len(t.shape) >= 2:
                batch = 1
                for s in t.shape[:-2]:
                    batch *= s
                m, n = sorted(t.shape[-2:])
                total += batch * opt_ns_iters(opt) * (4.0 * m * m * n + 2.0 * m * m * m) + 6.0 * t.numel
            else:
                total += 12.0 * t.numel
    return total


def opt_ns_iters(opt) -> int:
    return getattr(getattr(opt, "muon", opt), "ns_iters", 5)


def round_compute_flops(am, stats) -> Tuple[float, float]:
    """(recompute FLOPs chosen by the plan, always-on flash-backward rescan FLOPs)."""
    return float(stats.recompute_flops), 0.5 * float(stats.attn_fwd_flops)


def step_flops_breakdown(am, stats, mode: str = "full") -> Tuple[float, float]:
    """Returns ``(effective, hardware)`` FLOPs of one optimizer step on this rank."""
    f = fwd_flops(am, stats)
    h = head_flops(am, stats.tokens)
    eff = f + bwd_flops(am, stats, mode) + (3.0 * h if mode == "full" else 2.0 * h) + opt_flops_per_step(am)
    rec, rescan = round_compute_flops(am, stats)
    return eff, eff + rec + rescan
