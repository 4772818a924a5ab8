"""Loss-curve parity harness (flextrain/bench/parity.py:67-893, flextrain/bench/README.md:45-66).

Trains the same randomly initialised model twice on the same token stream — once with a naive autograd PyTorch
implementation + ``torch.optim.AdamW`` and once with the engine under a hand-forced working set — and reports the
windowed mean ``|Δloss|``.  Configurations: A all-on-device, B multi-chunk, C multi-round, D host offload (forced tier),
E weight ring, F gradient ring, G optimizer-state ring, H sequences that span chunks.

    python -m flextrain_b200.bench.parity --config all --steps 30 [--device cuda:0]
"""
from __future__ import annotations

import argparse
import json
import sys
from dataclasses import dataclass

import torch

import flextrain_b200 as ft
from flextrain_b200.bench.naive import clone_params, naive_loss
from flextrain_b200.engine.host_memory import UnpinnedHostBackend

DIMS = dict(vocab_size=2048, n_layers=4, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, expert_dim=704)
SEQ, BATCH = 128, 1024

CONFIGS = {
    "A": dict(),
    "B": dict(chunk=256),
    "C": dict(chunk=256, round_tokens=512),
    "D": dict(chunk=256, host_act_buffer_size=256 << 20, _force=0),
    "E": dict(n_gpu_layers=2),
    "F": dict(n_gpu_grads=2, chunk=256, round_tokens=512),
    "G": dict(n_gpu_opt_layers=2),
    "H": dict(chunk=64, _max_seq=320, _seq_lens=[300, 100, 180, 128]),
}


def run_config(name: str, steps: int, device: str, lr: float = 5e-4, window: int = 10) -> dict:
    kw = dict(CONFIGS[name])
    force, max_seq, seq_lens = kw.pop("_force", None), kw.pop("_max_seq", SEQ), kw.pop("_seq_lens", SEQ)
    dt = torch.bfloat16 if device.startswith("cuda") else torch.float32
    ws = ft.WorkingSetConfig.simple(max_seq_len=max_seq, max_global_batch_tokens=BATCH, **kw)
    am = ft.from_dims(DIMS, arch="llama", optimizer=ft.AdamW(lr=lr, state_dtype=torch.float32), max_seq_len=max_seq,
                      max_global_batch_tokens=BATCH, max_gpu_mem_bytes=16 << 30, max_host_mem_bytes=16 << 30,
                      device=device, compute_dtype=dt, master_dtype=dt, grad_dtype=dt, working_set=ws,
                      force_saved_act_level=force,
                      host_backend=None if device.startswith("cuda") else UnpinnedHostBackend())
    P = clone_params(am)
    P = {k: v.detach().cpu().requires_grad_(True) for k, v in P.items()}
    opt = torch.optim.AdamW(list(P.values()), lr=lr, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0)
    src = ft.SyntheticTokenSource(DIMS["vocab_size"], seq_lens, seed=17)
    diffs, le, ln = [], [], []
    cpu_view = _CPUView(am)
    for _ in range(steps):
        seqs = src.get_sequences(BATCH)
        opt.zero_grad()
        loss = naive_loss(cpu_view, P, seqs)
        loss.backward()
        opt.step()
        st = am.fwd_bwd(seqs)
        am.step()
        le.append(st.loss); ln.append(float(loss.detach()))
        diffs.append(abs(st.loss - float(loss.detach())))
    win = [sum(diffs[i:i + window]) / len(diffs[i:i + window]) for i in range(0, len(diffs), window)]
    return {"config": name, "max_windowed_abs_dloss": max(win), "final_engine": le[-1], "final_naive": ln[-1]}


@dataclass
class LossCurveParityConfig:
    """One run of the harness (the reference's record of the same name, flextrain/bench/parity.py): which forced
    working set (``CONFIGS`` key), how many steps, where."""
    config: str = "A"
    steps: int = 30
    device: str = "cpu"
    lr: float = 5e-4
    window: int = 10
    tolerance: float = 0.06              # bound on the windowed mean |engine loss - naive loss|


@dataclass
class LossCurveParityResult:
    config: str
    max_windowed_abs_dloss: float
    final_engine: float
    final_naive: float
    passed: bool


def run_loss_curve_parity(cfg: LossCurveParityConfig) -> LossCurveParityResult:
    r = run_config(cfg.config, cfg.steps, cfg.device, cfg.lr, cfg.window)
    return LossCurveParityResult(r["config"], r["max_windowed_abs_dloss"], r["final_engine"], r["final_naive"],
                                 r["max_windowed_abs_dloss"] <= cfg.tolerance)


class _CPUView:
    """Lets the naive model read the engine's layer objects (configs, scales) without touching its buffers."""

    def __init__(self, am):
        self.layers, self.embed, self.head = am.layers, am.embed, am.head


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="all")
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--device", default="cuda:0" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--tolerance", type=float, default=0.10)
    a = ap.parse_args(argv)
    names = list(CONFIGS) if a.config == "all" else a.config.split(",")
    worst = 0.0
    for n in names:
        r = run_config(n, a.steps, a.device)
        worst = max(worst, r["max_windowed_abs_dloss"])
        print(json.dumps(r))
    print(f"worst windowed |dloss| = {worst:.4f} (tolerance {a.tolerance})")
    return 0 if worst <= a.tolerance else 1


if __name__ == "__main__":
    sys.exit(main())
