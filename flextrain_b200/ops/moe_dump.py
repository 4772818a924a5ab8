"""Dump-and-diff diagnostics for MoE layers (the reference's ``FLEXTRAIN_MOE_DUMP_DIR``, flextrain/ops/_moe_dump.py).

With ``FTB_MOE_DUMP_DIR=<dir>`` every MoE forward writes its router logits, routing weights, chosen experts and block
output to ``<dir>/call<k>.pt`` (``k`` counts MoE forwards of the process; a rank suffix is added in multi-rank jobs).
Two runs that should agree — a code change, another back end, another parallel layout on the same data — are then
compared with :func:`diff_dumps` (also ``python -m flextrain_b200.ops.moe_dump DIR_A DIR_B``).  Off by default: the
environment variable is read once, at import."""
from __future__ import annotations

import os
import sys
from typing import Dict, List

import torch

DUMP_DIR = os.environ.get("FTB_MOE_DUMP_DIR") or None
_calls = 0


def enabled() -> bool:
    return DUMP_DIR is not None


def dump(**tensors) -> None:
    """Write one MoE forward's tensors (no-op unless dumping is on)."""
    global _calls
    if DUMP_DIR is None:
        return
    os.makedirs(DUMP_DIR, exist_ok=True)
    rank = os.environ.get("RANK")
    name = f"call{_calls:06d}" + (f"_rank{int(rank)}" if rank is not None and os.environ.get("WORLD_SIZE", "1") != "1" else "")
    torch.save({k: v.detach().to("cpu") for k, v in tensors.items() if v is not None}, os.path.join(DUMP_DIR, name + ".pt"))
    _calls += 1


def diff_dumps(dir_a: str, dir_b: str) -> List[Dict]:
    """Per call and tensor: max abs difference, relative L2 difference and, for expert choices, the fraction of rows
    whose expert set differs."""
    rows = []
    names = sorted(set(os.listdir(dir_a)) & set(os.listdir(dir_b)))
    for n in names:
        a, b = torch.load(os.path.join(dir_a, n)), torch.load(os.path.join(dir_b, n))
        for k in sorted(set(a) & set(b)):
            x, y = a[k], b[k]
            if x.shape != y.shape:
                rows.append({"call": n, "tensor": k, "shape_a": list(x.shape), "shape_b": list(y.shape)})
                continue
            if k == "chosen_experts":
                same = (x.sort(-1).values == y.sort(-1).values).all(-1)
                rows.append({"call": n, "tensor": k, "rows_with_other_experts": float((~same).float().mean())})
                continue
            xf, yf = x.float(), y.float()
            rows.append({"call": n, "tensor": k, "max_abs": float((xf - yf).abs().max()) if xf.numel() else 0.0,
                         "rel_l2": float((xf - yf).norm() / (yf.norm() + 1e-12))})
    return rows


if __name__ == "__main__":
    for r in diff_dumps(sys.argv[1], sys.argv[2]):
        print(r)
