"""Authoritative FLOP accounting (flextrain/core/flop_accounting.py:111-460, train.py:110-151).

effective = forward + backward (2x forward for full fine-tuning, 1x for LoRA: no base weight gradients)
            + head (forward + 2 backward GEMMs) + optimizer;
hardware  = effective + recompute chosen by the save-level plan + 0.5 x attention forward (the flash
            backward re-scans the scores).
"""
from __future__ import annotations

from typing import Tuple


def _sequence_fwd_flops(am, seq_len: int) -> float:
    """Forward FLOPs of ONE sequence of ``seq_len`` tokens through every layer and the head: each layer's own
    ``compute_cost`` at the causal mean context ``seq_len / 2`` (flextrain/core/flop_accounting.py:111-137)."""
    n = int(seq_len)
    return float(sum(layer.compute_cost(n, n / 2).total_fwd_flops for layer in am.layers)) + head_flops(am, n)


def fwd_flops(am, stats) -> float:
    """Forward FLOPs of what ``stats`` (a :class:`StepStats`) recorded, or, given a sequence length instead (the
    reference's form), of one sequence of that length including the head."""
    if isinstance(stats, (int, float)):
        return _sequence_fwd_flops(am, int(stats))
    return float(stats.fwd_flops)


def head_flops(am, tokens: int) -> float:
    return 2.0 * tokens * am.head.vocab_size * am.head.d_model


def bwd_flops(am, stats, mode: str = "full") -> float:
    if mode not in ("full", "lora"):
        raise ValueError(f"mode must be 'full' or 'lora', got {mode!r}")
    return (2.0 if mode == "full" else 1.0) * fwd_flops(am, stats)


def step_flops(am, seq_lens, *, mode: str = "full") -> float:
    """FLOPs of one optimizer step over sequences of the given lengths: forward + backward per sequence (the
    attention term is not linear in length, so they are summed one by one) + the optimizer
    (flextrain/core/flop_accounting.py:303-320)."""
    return float(sum(fwd_flops(am, int(n)) + bwd_flops(am, int(n), mode) for n in seq_lens)) + opt_flops_per_step(am)


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
