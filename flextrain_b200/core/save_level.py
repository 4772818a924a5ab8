"""Save-level planning: DP tables, native solver binding, and plan post-processing.

Mirrors flextrain/core/save_level.py (SaveLevel :57-80, HardwareCost :88-132, build_dp_tables
:242-301, plan_from_solution :311-474) and the ctypes wrapper of the reference scheduler
(helpers/transmission_scheduler/transmission_scheduler/__init__.py:61-141).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

ON_DEVICE = -1


@dataclass(frozen=True)
class HardwareCost:
    """Throughput model used to turn FLOPs and bytes into milliseconds."""
    peak_tflops: float = 1362.7            # sustained bf16 GEMM rate
    pcie_bw_gbps: float = 50.0             # host <-> HBM, per direction
    nvlink_bw_gbps: float = 770.0          # peer HBM <-> HBM, per direction
    mem_bw_gbps: float = 6546.0
    practical_efficiency_factor: float = 1.0   # scales a nameplate peak down; 1.0 for a measured rate

    @property
    def effective_flops_per_ms(self) -> float:
        return self.practical_efficiency_factor * self.peak_tflops * 1e12 / 1e3

    @property
    def pcie_bytes_per_ms(self) -> float:
        return self.pcie_bw_gbps * 1e9 / 1e3

    def flops_to_ms(self, flops: float) -> float:
        rate = self.effective_flops_per_ms
        return flops / rate if rate > 0 else 0.0

    def bytes_to_ms(self, nbytes: float, link: str = "pcie") -> float:
        bw = {"pcie": self.pcie_bw_gbps, "nvlink": self.nvlink_bw_gbps, "hbm": self.mem_bw_gbps}[link]
        return nbytes / (bw * 1e9) * 1e3


@dataclass
class SaveLevelPlan:
    """``levels[(layer, chunk)]`` = tier saved to the host, or ``ON_DEVICE``."""
    levels: Dict[Tuple[int, int], int]
    n_layers: int
    n_chunks: int
    host_bytes: int = 0
    recompute_flops: float = 0.0
    solver_value: float = 0.0
    feasible: bool = True

    @classmethod
    def all_on_device(cls, n_layers: int, n_chunks: int) -> "SaveLevelPlan":
        return cls({(l, c): ON_DEVICE for l in range(n_layers) for c in range(n_chunks)}, n_layers, n_chunks)

    @classmethod
    def uniform(cls, n_layers: int, n_chunks: int, level: int) -> "SaveLevelPlan":
        return cls({(l, c): level for l in range(n_layers) for c in range(n_chunks)}, n_layers, n_chunks)

    def level(self, layer: int, chunk: int) -> int:
        return self.levels[(layer, chunk)]

    # the reference's spellings (flextrain/core/save_level.py:88-132)
    def level_for(self, layer_id: int, chunk_id: int) -> int:
        return self.levels[(layer_id, chunk_id)]

    @property
    def choices(self) -> Dict[Tuple[int, int], int]:
        return self.levels

    def histogram(self) -> Dict[int, int]:
        h: Dict[int, int] = {}
        for v in self.levels.values():
            h[v] = h.get(v, 0) + 1
        return h


@dataclass
class DPTables:
    compute_ms: np.ndarray      # (T,)
    dur_ms: np.ndarray          # (T, k)
    value_ms: np.ndarray        # (T, k)
    bytes_: np.ndarray          # (T, k) offloaded bytes per option
    valid_k: np.ndarray         # (T,)
    tasks: List[Tuple[int, int]]


def build_dp_tables(layers, chunk_tokens: Sequence[int], hw: HardwareCost, *, avg_ctx: Optional[Sequence[float]] = None,
                    link: str = "pcie", k: int = 4) -> DPTables:
    """Rectangular ``(T, k)`` tables in forward task order (``for layer: for chunk``)."""
    tasks, comp, dur, val, byt, vk = [], [], [], [], [], []
    for li, layer in enumerate(layers):
        schema = layer.activation_schema
        for ci, ntok in enumerate(chunk_tokens):
            cost = layer.compute_cost(ntok, (avg_ctx[ci] if avg_ctx is not None else ntok / 2))
            tasks.append((li, ci))
            comp.append(hw.flops_to_ms(cost.total_fwd_flops))
            nt = min(k, schema.max_tier + 1)
            d, v, b = [], [], []
            for L in range(k):
                LL = min(L, nt - 1)
                nb = schema.home_size_bytes(ntok, LL)
                b.append(nb)
                d.append(hw.bytes_to_ms(nb, link))
                v.append(hw.flops_to_ms(cost.avoided_recompute_flops[LL]))
            dur.append(d); val.append(v); byt.append(b); vk.append(nt)
    return DPTables(np.asarray(comp, dtype=np.float64), np.asarray(dur, dtype=np.float64),
                    np.asarray(val, dtype=np.float64), np.asarray(byt, dtype=np.int64),
                    np.asarray(vk, dtype=np.int32), tasks)


class TransmissionScheduler:
    """Binding to ``csrc/dp_solver.cpp``; ``solve`` returns per-task tiers or ``None`` when infeasible."""

    def __init__(self, tick_ms: float = 0.1, force_scalar: bool = False):
        from ..ops.cuda import load
        self.lib = load("dp_solver")
        self.lib.ftb_dp_solve.restype = ctypes.c_double
        self.tick_ms = tick_ms
        self.force_scalar = force_scalar

    def solve(self, compute_ms, dur_ms, value_ms, n_slots: int, pinned=None, valid_k=None):
        compute_ms = np.ascontiguousarray(compute_ms, dtype=np.float64)
        dur_ms = np.ascontiguousarray(dur_ms, dtype=np.float64)
        value_ms = np.ascontiguousarray(value_ms, dtype=np.float64)
        T, k = dur_ms.shape
        pinned = np.zeros(T, dtype=np.uint8) if pinned is None else np.ascontiguousarray(pinned, dtype=np.uint8)
        valid_k = np.full(T, k, dtype=np.int32) if valid_k is None else np.ascontiguousarray(valid_k, dtype=np.int32)
        out = np.empty(T, dtype=np.int32)
        total = float(compute_ms.sum())
        tick = max(self.tick_ms, total / float(1 << 20))
        # the table is T x window bytes: coarsen the tick until it stays under ~48 MB
        if n_slots >= 2 and T > n_slots:
            c = np.concatenate([[0.0], np.cumsum(compute_ms)])
            span = n_slots - 2
            window_ms = float((c[span + 1:] - c[1:T - span + 1]).max()) if span < T else total
            tick = max(tick, window_ms * T / 48e6)
        p = lambda a, t: a.ctypes.data_as(ctypes.POINTER(t))
        best = self.lib.ftb_dp_solve(ctypes.c_int(T), ctypes.c_int(k), ctypes.c_int(n_slots),
                                     p(compute_ms, ctypes.c_double), p(dur_ms, ctypes.c_double),
                                     p(value_ms, ctypes.c_double), p(pinned, ctypes.c_uint8),
                                     p(valid_k, ctypes.c_int32), ctypes.c_double(tick), p(out, ctypes.c_int32),
                                     ctypes.c_int(1 if self.force_scalar else 0))
        if best < 0:
            return None, -1.0
        return out, best


def solve_reference(compute_ms, dur_ms, value_ms, n_slots: int, pinned=None, tick_ms: float = 0.1):
    """Pure-Python statement of the same DP (small problems; used by tests to cross-check the native solver)."""
    T, k = np.asarray(dur_ms).shape
    pinned = [0] * T if pinned is None else list(pinned)
    c = [0]
    acc = 0.0
    for t in range(T):
        acc += compute_ms[t]
        c.append(int(round(acc / tick_ms)))
    INF = 1 << 60
    states = {0: (0.0, [])}
    for t in range(T):
        last = t + n_slots - 2
        deadline = (c[last + 1] - c[t + 1]) if (n_slots >= 2 and last < T - 1) else (0 if n_slots < 2 else INF)
        gap = (c[t + 2] - c[t + 1]) if t + 1 < T else 0
        new = {}
        for s, (val, path) in states.items():
            if pinned[t]:
                opts = [(-1, 0, max(value_ms[t]))]
            else:
                opts = [(L, int(np.ceil(dur_ms[t][L] / tick_ms - 1e-9)), value_ms[t][L]) for L in range(k)]
            for L, d, v in opts:
                fin = s + d
                if L >= 0 and fin > deadline:
                    continue
                s2 = max(0, fin - gap)
                cand = val + v
                if s2 not in new or cand > new[s2][0]:
                    new[s2] = (cand, path + [L])
        states = new
        if not states:
            return None, -1.0
    best = max(states.values(), key=lambda x: x[0])
    return np.asarray(best[1], dtype=np.int32), best[0]


def plan_from_solution(tables: DPTables, solution: Optional[np.ndarray], n_layers: int, n_chunks: int, *,
                       n_gpu_act_slots: int, host_budget_bytes: Optional[int] = None,
                       force_level: Optional[int] = None) -> SaveLevelPlan:
    """Turn solver output into a plan (flextrain/core/save_level.py:311-474):
    infeasible → all tier 0; clamp to each task's valid tiers; the last ``n_gpu_act_slots`` tasks stay on
    device; if the host bytes exceed the budget demote 3→2→1 first, then 1→0, least value per byte first."""
    T = len(tables.tasks)
    feasible = solution is not None
    lv = np.zeros(T, dtype=np.int64) if solution is None else np.asarray(solution, dtype=np.int64).copy()
    if force_level is not None:
        lv[:] = force_level
    lv = np.minimum(lv, tables.valid_k - 1)
    tail = max(0, T - n_gpu_act_slots)
    lv[tail:] = ON_DEVICE
    if solution is not None:
        lv[np.asarray(solution) < 0] = ON_DEVICE
        lv[tail:] = ON_DEVICE

    def host_bytes() -> int:
        return int(sum(tables.bytes_[t, lv[t]] for t in range(T) if lv[t] >= 0))

    if host_budget_bytes is not None and host_bytes() > host_budget_bytes:
        for floor in (1, 0):
            while host_bytes() > host_budget_bytes:
                cands = [t for t in range(T) if lv[t] > floor]
                if not cands:
                    break

                def loss_per_byte(t):
                    L = lv[t]
                    dv = tables.value_ms[t, L] - tables.value_ms[t, L - 1]
                    db = max(1, tables.bytes_[t, L] - tables.bytes_[t, L - 1])
                    return dv / db
                t = min(cands, key=loss_per_byte)
                lv[t] -= 1
        if host_bytes() > host_budget_bytes:
            raise ValueError(f"host activation budget too small: tier-0 state needs {host_bytes()} bytes, "
                             f"budget is {host_budget_bytes}")
    levels = {tables.tasks[t]: int(lv[t]) for t in range(T)}
    return SaveLevelPlan(levels, n_layers, n_chunks, host_bytes=host_bytes(), feasible=feasible)
