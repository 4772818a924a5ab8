"""Dims-only byte / FLOP estimators and divisor helpers (flextrain/core/_sizing.py:49-293)."""
from __future__ import annotations

from typing import Dict, List

_B = {"bfloat16": 2, "float16": 2, "float32": 4}


def divisors(n: int) -> List[int]:
    out = set()
    i = 1
    while i * i <= n:
        if n % i == 0:
            out.add(i); out.add(n // i)
        i += 1
    return sorted(out)


def prev_high_div(n: int, quantum: int = 1024) -> int:
    """Largest value <= n that is a multiple of ``quantum`` and has many divisors (prefers powers of two times
    small odd factors), so that a global batch splits into equal rounds and chunks with no tail."""
    if n <= quantum:
        return max(n, 1)
    best, best_score = quantum, -1
    lo = max(quantum, int(n * 0.75))
    m = n // quantum * quantum
    while m >= lo:
        score = len(divisors(m // quantum))
        if score > best_score:
            best, best_score = m, score
        m -= quantum
    return best


def layer_param_count(d: Dict) -> int:
    """Parameters of one decoder layer from a dims dict (dense or MoE)."""
    dm, hd = d["d_model"], d["head_dim"]
    q, kv = d["n_heads"] * hd, d["n_kv_heads"] * hd
    attn = dm * (q + 2 * kv) + q * dm
    E = d.get("num_routed_experts", 0) or 0
    F = d["expert_dim"]
    if E > 0:
        ffn = E * 3 * dm * F + dm * E + (d.get("num_shared_experts", 0) or 0) * 3 * dm * d.get("shared_dim", F)
    else:
        ffn = 3 * dm * F
    return attn + ffn + 2 * dm


def model_param_count(d: Dict) -> int:
    return d["n_layers"] * layer_param_count(d) + 2 * d["vocab_size"] * d["d_model"] + d["d_model"]


def matmul_flops_per_token(d: Dict, active_only: bool = True) -> float:
    """Forward GEMM FLOPs per token of the whole model (excluding attention score/value products)."""
    dm, hd = d["d_model"], d["head_dim"]
    q, kv = d["n_heads"] * hd, d["n_kv_heads"] * hd
    per_layer = 2.0 * (dm * (q + 2 * kv) + q * dm)
    E = d.get("num_routed_experts", 0) or 0
    F = d["expert_dim"]
    if E > 0:
        k = d.get("top_k", 1) if active_only else E
        per_layer += 2.0 * (k * 3 * dm * F + dm * E)
    else:
        per_layer += 2.0 * 3 * dm * F
    return d["n_layers"] * per_layer + 2.0 * dm * d["vocab_size"]


def tier0_bytes_per_token(d: Dict, act_bytes: int = 2) -> int:
    """Residual input + K + V per layer: what must survive per (layer, token) at save level 0."""
    return (d["d_model"] + 2 * d["n_kv_heads"] * d["head_dim"]) * act_bytes + 8
