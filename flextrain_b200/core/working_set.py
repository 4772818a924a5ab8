"""Working-set planner: where every parameter, gradient, optimizer-state and activation byte lives.

Follows the reference's ``determine_working_set_config`` (flextrain/core/working_set.py:664-1366;
chunk search :1369-1786) — budgets minus leeway, spec-driven model memory, compute-bound round size,
tier-0 cap, highly-divisible rounding, arithmetic-intensity floor for the chunk, a candidate search
with a "healthy" rule — and extends it from one GPU to an NVSwitch box:

* a **shard dimension**: ``none`` (replicated), ``opt``, ``opt+grad``, ``opt+grad+param`` — each level
  divides that state class by the data-parallel world size and adds NVLink traffic
  (reduce-scatter of gradients, all-gather of parameters) costed at ``bytes / nvlink_bw``;
* host offload stays available per state class, costed at ``bytes / pcie_bw``;
* the planner picks the candidate with the smallest estimated step time among those that fit,
  and keeps a per-candidate trace so the decision can be explained (``plan.report``).

With ``world_size == 1`` the shard dimension collapses and the search is the reference's:
ring sizes ``n_gpu_layers / n_gpu_grads / n_gpu_opt_layers`` and activation slots under the byte budgets.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

from .save_level import HardwareCost
from ._sizing import divisors

GiB = 1 << 30
# Data-parallel state sharding.  There is no "optimizer state only" level: the gradient reduction of the peer-memory
# path IS a reduce-scatter into an fp32 shard, so sharded gradients come for free with a sharded optimizer.
SHARD_MODES = ("none", "opt+grad", "opt+grad+param")
RING_DEPTHS = (2, 3, 4)       # GPU slots of a state class whose master copy lives in host memory


@dataclass
class WorkingSetConfig:
    """Planner output (flextrain/core/working_set.py:91-129) plus the parallel layout."""
    target_round_tokens: int
    max_chunk_size: int
    max_training_chunks: int
    max_total_round_tokens: int
    target_num_rounds: int
    n_gpu_layers: Optional[int]            # None = all layers resident
    n_gpu_grads: Optional[int]
    n_gpu_opt_layers: Optional[int]
    n_gpu_act_slots: Optional[int] = None  # (layer, chunk) activation sets kept in HBM; None = derived from the ring bytes
    gpu_act_buffer_size: int = 0
    host_act_buffer_size: int = 0
    max_seq_len: int = 0
    max_global_batch_tokens: Optional[int] = None          # None = target_round_tokens x target_num_rounds
    # parallel layout
    world_size: int = 1
    shard: str = "none"
    tp: int = 1
    ep: int = 1
    # estimates (ms per optimizer step) and the search trace
    est_step_ms: float = 0.0
    est_compute_ms: float = 0.0
    est_pcie_ms: float = 0.0
    est_nvlink_ms: float = 0.0
    healthy: bool = True
    head_chunk_size: Optional[int] = None      # set when the planner had to shrink the head's logits micro-chunk
    report: List[str] = field(default_factory=list)
    # what the plan was made for: informational, and what a hand-built configuration in the reference's form carries
    # (flextrain/core/working_set.py:91-129)
    available_gpu_memory_bytes: int = 0
    available_host_memory_bytes: int = 0
    leeway_gpu_memory_bytes: int = 0
    leeway_host_memory_bytes: int = 0
    hardware_env: Optional[dict] = None
    raw: Optional[dict] = None

    def __post_init__(self):
        if self.max_global_batch_tokens is None:
            self.max_global_batch_tokens = int(self.target_round_tokens) * max(int(self.target_num_rounds), 1)
        if not self.max_seq_len:
            self.max_seq_len = int(self.max_chunk_size)

    def resolve_act_slots(self, layers) -> None:
        """A hand-built configuration may give the activation ring in bytes only: turn it into a slot count with the
        largest per-layer activation set at ``max_chunk_size`` (no ring bytes = everything stays in HBM)."""
        if self.n_gpu_act_slots is not None:
            return
        per_slot = max((l.activation_schema.device_size_bytes(self.max_chunk_size) for l in layers), default=0)
        if self.gpu_act_buffer_size <= 0 or per_slot <= 0:
            self.n_gpu_act_slots = 1 << 30
        else:
            self.n_gpu_act_slots = max(2, int(self.gpu_act_buffer_size // per_slot))

    @classmethod
    def simple(cls, *, max_seq_len: int, max_global_batch_tokens: int, chunk: Optional[int] = None,
               round_tokens: Optional[int] = None, n_layers: int = 1, **kw) -> "WorkingSetConfig":
        """Hand-built config that forces a code path (used by tests and the parity harness)."""
        chunk = chunk or max_seq_len
        round_tokens = round_tokens or max_global_batch_tokens
        n_chunks = max(1, math.ceil(round_tokens / chunk) + 1)
        base = dict(target_round_tokens=round_tokens, max_chunk_size=chunk, max_training_chunks=4 * n_chunks,
                    max_total_round_tokens=max(round_tokens, max_seq_len), target_num_rounds=max(
                        1, math.ceil(max_global_batch_tokens / round_tokens)), n_gpu_layers=None, n_gpu_grads=None,
                    n_gpu_opt_layers=None, n_gpu_act_slots=1 << 30, gpu_act_buffer_size=0, host_act_buffer_size=0,
                    max_seq_len=max_seq_len, max_global_batch_tokens=max_global_batch_tokens)
        base.update(kw)
        return cls(**base)


@dataclass
class ModelMemory:
    """Spec-driven byte totals (flextrain/core/working_set.py:172-373)."""
    layer_param: List[int]
    layer_master: List[int]
    layer_grad: List[int]
    layer_opt: List[int]
    embed_head_resident: int
    act_full_per_token: List[int]       # device slot bytes per token at full tier, per layer
    act_tier_per_token: List[List[int]]  # [layer][tier]
    fwd_flops_per_token: float
    head_flops_per_token: float
    # share of the layers' forward FLOPs that has to be recomputed in backward when only tiers <= k were saved,
    # from every layer's ``ComputeCost.avoided_recompute_flops`` (index k; the last entry is 0: everything saved)
    recompute_frac: List[float] = field(default_factory=lambda: [0.0])

    @property
    def n_layers(self) -> int:
        return len(self.layer_param)


def baseline_model_memory(layers, embed, head, optimizer, probe_tokens: int = 4096) -> ModelMemory:
    from ..engine.buffers import LayerBuffers
    lp, lm, lg, lo, af, at = [], [], [], [], [], []
    flops = 0.0
    n_tiers = max((l.activation_schema.max_tier for l in layers), default=0) + 1
    redo = [0.0] * n_tiers
    for layer in layers:
        lb = LayerBuffers(layer.param_spec, optimizer)
        lp.append(lb.p_bytes); lm.append(lb.m_bytes); lg.append(lb.g_bytes); lo.append(lb.o_bytes)
        sch = layer.activation_schema
        af.append(math.ceil(sch.device_size_bytes(probe_tokens) / probe_tokens))
        at.append([math.ceil(sch.home_size_bytes(probe_tokens, L) / probe_tokens) for L in range(sch.max_tier + 1)])
        cost = layer.compute_cost(probe_tokens, probe_tokens / 2)
        flops += cost.total_fwd_flops / probe_tokens
        av = cost.avoided_recompute_flops
        for k in range(n_tiers):
            redo[k] += (av[-1] - av[min(k, len(av) - 1)]) / probe_tokens
    eh = 0
    for blk in (embed, head):
        lb = LayerBuffers(blk.param_spec, optimizer)
        eh += lb.p_bytes + lb.g_bytes + lb.o_bytes
    head_flops = 2.0 * head.vocab_size * head.d_model
    return ModelMemory(lp, lm, lg, lo, eh, af, at, flops, head_flops, [r / max(flops, 1e-9) for r in redo])


def _workspace_bytes(layers, head, chunk: int, act_bytes: int = 2, head_rows: Optional[int] = None) -> int:
    """Transient GPU memory while one chunk is in flight: residual stream in/out, the widest projection output
    and its gradient, attention workspace, and one head micro-chunk of logits."""
    widest = 0
    d = 0
    for l in layers:
        c = l.cfg
        d = c.d_model
        w = 0
        if c.attn is not None:
            w = max(w, (c.attn.q_dim * (2 if c.attn.gated else 1) + 2 * c.attn.kv_dim))
        if c.ffn is not None:
            w = max(w, 3 * c.ffn.ffn_dim)
        if c.moe is not None:
            w = max(w, 3 * c.moe.expert_dim * c.moe.top_k + 3 * c.moe.shared_dim)
        widest = max(widest, w)
    per_tok = (4 * d + 2 * widest) * act_bytes
    head_ws = min(chunk, head_rows or head.head_chunk_size) * head.vocab_size * act_bytes * 2
    return chunk * per_tok + head_ws + (256 << 20)


def determine_working_set_config(*, layers, embed, head, optimizer, max_seq_len: int, max_global_batch_tokens: int,
                                 max_gpu_mem_bytes: int, max_host_mem_bytes: int,
                                 leeway_gpu_mem_bytes: int = 3 * GiB, leeway_host_mem_bytes: int = 4 * GiB,
                                 hw: Optional[HardwareCost] = None, world_size: int = 1, tp: int = 1, ep: int = 1,
                                 shard: Optional[str] = None, min_chunk_size: Optional[int] = None,
                                 max_chunk_size: Optional[int] = None, force_saved_act_level: Optional[int] = None,
                                 verbose: bool = False, layers_are_local: bool = False,
                                 opt_state: str = "auto") -> WorkingSetConfig:
    """``opt_state``: ``"auto"`` lets the search decide where optimizer state lives, ``"host"`` restricts it to the
    layouts that stream the state through pinned host memory, ``"device"`` to the ones that keep it in HBM."""
    hw = hw or HardwareCost()
    if opt_state not in ("auto", "host", "device"):
        raise ValueError(f"opt_state must be auto, host or device, not {opt_state!r}")
    log: List[str] = []

    def say(msg: str):
        log.append(msg)
        if verbose:
            print(f"[Working Set Log] {msg}")

    # 1. budgets
    gpu_budget = max_gpu_mem_bytes - leeway_gpu_mem_bytes
    host_budget = max(0, max_host_mem_bytes - leeway_host_mem_bytes)
    if gpu_budget <= 0:
        raise ValueError(f"GPU budget {max_gpu_mem_bytes / GiB:.1f} GiB is below the leeway "
                         f"{leeway_gpu_mem_bytes / GiB:.1f} GiB")
    dp = max(1, world_size // max(tp, 1) // 1)
    say(f"budgets: gpu {gpu_budget / GiB:.1f} GiB, host {host_budget / GiB:.1f} GiB, world {world_size} "
        f"(dp {dp}, tp {tp}, ep {ep})")

    # 2. model memory
    mm = baseline_model_memory(layers, embed, head, optimizer)
    L = mm.n_layers
    tp_group = tp
    if layers_are_local:
        tp = 1          # the layers already describe one rank's part: sizes and FLOPs below are per rank as they are
    P, G, O = sum(mm.layer_param) // tp, sum(mm.layer_grad) // tp, sum(mm.layer_opt) // tp
    say(f"model: {L} layers, params {P / GiB:.2f} GiB, grads {G / GiB:.2f} GiB, opt {O / GiB:.2f} GiB per TP rank, "
        f"embed+head resident {mm.embed_head_resident / GiB:.2f} GiB")
    batch_per_rank = max(max_seq_len, max_global_batch_tokens // dp)
    flops_tok = (mm.fwd_flops_per_token + mm.head_flops_per_token) / tp
    compute_ms_step = hw.flops_to_ms(3.0 * flops_tok * batch_per_rank)

    # 3. compute-bound round size: one layer's compute must cover its weight-in + grad-out PCIe time
    layer_bytes = max(mm.layer_param) + max(mm.layer_grad)
    layer_flops_tok = 3.0 * mm.fwd_flops_per_token / max(L, 1)
    tokens_compute_bound = int(hw.bytes_to_ms(layer_bytes, "pcie") / max(hw.flops_to_ms(layer_flops_tok), 1e-12))
    # 4. arithmetic-intensity floor for a chunk: GEMM (T x K x N) is compute-bound once T >= peak / mem_bw
    ai_floor = int(2 * hw.peak_tflops * 1e12 / (hw.mem_bw_gbps * 1e9) / 2)
    lo_chunk = min_chunk_size or min(max(1024, ai_floor), max(1024, batch_per_rank))
    hi_chunk = max_chunk_size or 16384
    full_tok = sum(mm.act_full_per_token)
    tier0_tok = sum(a[0] for a in mm.act_tier_per_token)

    n_tiers = len(mm.recompute_frac)
    tier_tok = [sum(a[min(k, len(a) - 1)] for a in mm.act_tier_per_token) for k in range(n_tiers)]

    # Host residency of a state class is what a single GPU does when HBM is short.  With several ranks the states are
    # sharded over the ranks first; the one multi-rank layout that also streams optimizer state through the host is a
    # model-parallel group that spans the job (each rank updates its own slice of every matrix from pinned host state,
    # layer by layer) or the library-collective back end (which keeps the single-GPU rings).
    import os as _os
    multi_host_ok = world_size > 1 and (tp_group == world_size or _os.environ.get("FTB_DP_BACKEND") == "collective")

    best: Optional[Tuple[float, WorkingSetConfig]] = None
    # With dp > 1 the engine always reduce-scatters gradients into an fp32 shard and runs the optimizer on the
    # shard ("opt+grad"); "opt+grad+param" additionally defers the parameter all-gather to first use.
    modes = [shard] if shard is not None else (("opt+grad", "opt+grad+param") if dp > 1 else ("none",))
    # The head holds one micro-chunk of logits (rows x vocab) at a time.  On a tight budget that block is the largest
    # transient: if nothing fits with the configured micro-chunk the search is repeated with 1024 rows (the
    # reference's default, flextrain/nn/head.py:202-207) and the plan carries the smaller value.
    head_rows_options = [None] + ([1024] if head.head_chunk_size > 1024 else [])

    def search(head_rows: Optional[int]) -> None:
        nonlocal best
        for mode in modes:
            # "opt+grad+param" defers the parameter all-gather to the first GEMM that uses a layer (it overlaps the forward
            # pass instead of closing the optimizer step); the arena stays full size, so memory equals "opt+grad"
            p = P
            # local bf16 gradients stay full-size while rounds accumulate; the reduced fp32 shard is 2x bytes / dp
            g = G + (2 * G / dp if (dp > 1 and mode != "none") else 0)
            o = O / dp if mode != "none" else O
            # optimizer update traffic through HBM (params r/w, grads r, state r/w)
            opt_ms = hw.bytes_to_ms((2 * P + G + 2 * O) / (dp if mode != "none" else 1), "hbm")
            # NVLink traffic per step and rank: gradient reduce-scatter (+ all-gather of the reduced grads when not
            # sharded), parameter all-gather after the sharded update
            nv = 0.0
            if dp > 1:
                f = (dp - 1) / dp
                nv += G * f                                   # reduce-scatter
                nv += (G * f) if mode == "none" else (P * f)  # all-gather grads, or updated params
            nv_ms = hw.bytes_to_ms(nv, "nvlink")
            # "opt+grad+param": the all-gather runs under the next forward pass, not at the end of the step
            nv_exposed = 0.5 * nv_ms if mode == "opt+grad+param" else nv_ms
            if world_size == 1:
                residencies = ("all", "opt_host", "opt_grad_host", "all_host")
            else:
                residencies = ("all", "opt_host") if multi_host_ok else ("all",)
            if opt_state == "host":
                residencies = tuple(r for r in residencies if r != "all")
                if not residencies:
                    raise ValueError("optimizer state in host memory needs one GPU, a model-parallel group that spans "
                                     "the job, or the library-collective data-parallel back end")
            elif opt_state == "device":
                residencies = ("all",)
            for resid in residencies:
                for depth in ((0,) if resid == "all" else RING_DEPTHS):
                    n_p = n_g = n_o = None
                    host_state = 0.0
                    pcie = 0.0
                    states = p + g + o
                    if resid != "all":
                        n_o = depth
                        states = p + g + depth * max(mm.layer_opt) / tp
                        host_state += o
                        pcie += 2 * o
                    if resid in ("opt_grad_host", "all_host"):
                        n_g = depth
                        states -= g - depth * max(mm.layer_grad) / tp
                        host_state += g
                    if resid == "all_host":
                        n_p = depth
                        states -= p - depth * max(mm.layer_param) / tp
                        host_state += p
                    if host_state > host_budget:
                        say(f"[{mode}/{resid}] host-bound: states need {host_state / GiB:.1f} GiB of host")
                        break
                    fixed = states + mm.embed_head_resident
                    # a deeper ring hides more of a layer's transfer behind the layers before it
                    exposure = 0.05 if depth == 0 else 0.10 / (depth - 1)
                    for chunk in _chunk_candidates(batch_per_rank, max_seq_len, lo_chunk, hi_chunk):
                        ws_b = _workspace_bytes(layers, head, chunk, head_rows=head_rows)
                        room = gpu_budget - fixed - ws_b
                        if room < full_tok * chunk / max(L, 1):
                            continue
                        # rounds that fit entirely on the device at full tier
                        r_dev = int(room // max(full_tok, 1))
                        rounds_pcie = 0.0
                        # a sequence is never split across rounds: a round holds at least one whole (longest) sequence
                        seq_floor = min(batch_per_rank, math.ceil(max_seq_len / chunk) * chunk)
                        tier_note = ""
                        if r_dev >= max(seq_floor, min(batch_per_rank, max(chunk, tokens_compute_bound if resid == "all_host"
                                                                          else chunk))):
                            round_tokens = _round_down_to_multiple(min(r_dev, batch_per_rank), chunk, batch_per_rank)
                            n_slots = 1 << 30
                            host_act = 0
                            recompute = 0.0
                        else:
                            # activations go to the host; the DP solver picks the tier per (layer, chunk) at run time.  For
                            # the estimate take the uniform tier with the smallest max(compute + recompute, PCIe): a higher
                            # tier moves more bytes but recomputes less (``recompute_frac`` from the layers' ComputeCost).
                            host_room = host_budget - host_state
                            n_slots = int(room // max(full_tok * chunk / max(L, 1), 1))
                            if n_slots < 2:
                                continue
                            pick = None
                            for k in range(n_tiers):
                                r_host = int(host_room // max(tier_tok[k], 1))
                                rt = _round_down_to_multiple(min(batch_per_rank, max(r_host, 0)), chunk, batch_per_rank)
                                if rt < max(chunk, seq_floor):
                                    continue
                                pc = 2.0 * tier_tok[k] * batch_per_rank
                                # forward is 1/3 of a step's layer FLOPs: recomputing a share r of it costs r/3 of the step
                                t_k = max(compute_ms_step * (1 + mm.recompute_frac[k] / 3), hw.bytes_to_ms(pc / 2, "pcie"))
                                if pick is None or t_k < pick[0]:
                                    pick = (t_k, k, rt, pc)
                            if pick is None:
                                continue
                            _, k_sel, round_tokens, rounds_pcie = pick
                            recompute = mm.recompute_frac[k_sel]
                            host_act = int(min(host_room, tier_tok[-1] * round_tokens))
                            tier_note = f" tier<={k_sel}"
                        n_rounds = math.ceil(batch_per_rank / round_tokens)
                        if resid == "all_host":
                            pcie_total = pcie + rounds_pcie + n_rounds * 2 * (p + g)
                        elif resid == "opt_grad_host":
                            pcie_total = pcie + rounds_pcie + n_rounds * 2 * g
                        else:
                            pcie_total = pcie + rounds_pcie
                        pcie_ms = hw.bytes_to_ms(pcie_total / 2, "pcie")      # both directions run concurrently
                        # optimizer state streams through the host while the update runs, after the last backward: that
                        # part of the traffic has no forward / backward compute to hide behind
                        opt_stream_ms = hw.bytes_to_ms(pcie / 2, "pcie") if resid != "all" else 0.0
                        # chunk-dependent efficiency: GEMMs below the arithmetic-intensity knee run memory-bound, and every
                        # (layer, chunk) pays its launches
                        n_chunks_step = math.ceil(batch_per_rank / chunk)
                        comp = compute_ms_step * (1 + recompute / 3) * (1 + ai_floor / (4.0 * chunk)) \
                            + 0.12 * n_chunks_step * L
                        # transfers overlap compute; what exceeds it is exposed
                        est = max(comp, pcie_ms - opt_stream_ms, nv_exposed) + exposure * pcie_ms + 0.05 * nv_ms \
                            + max(opt_ms, opt_stream_ms) + 2.0 * n_rounds
                        cfg = WorkingSetConfig(
                            target_round_tokens=round_tokens, max_chunk_size=chunk,
                            max_training_chunks=2 * math.ceil(round_tokens / chunk) + 2,
                            max_total_round_tokens=max(round_tokens, max_seq_len), target_num_rounds=n_rounds,
                            n_gpu_layers=n_p, n_gpu_grads=n_g, n_gpu_opt_layers=n_o, n_gpu_act_slots=n_slots,
                            gpu_act_buffer_size=int(room), host_act_buffer_size=host_act, max_seq_len=max_seq_len,
                            max_global_batch_tokens=max_global_batch_tokens, world_size=world_size, shard=mode, tp=tp_group,
                            ep=ep, est_step_ms=est, est_compute_ms=comp, est_pcie_ms=pcie_ms, est_nvlink_ms=nv_ms,
                            healthy=(n_slots >= 2), head_chunk_size=head_rows,
                            available_gpu_memory_bytes=int(max_gpu_mem_bytes),
                            available_host_memory_bytes=int(max_host_mem_bytes),
                            leeway_gpu_memory_bytes=int(leeway_gpu_mem_bytes),
                            leeway_host_memory_bytes=int(leeway_host_mem_bytes))
                        say(f"[{mode}/{resid}{'' if depth == 0 else '/ring ' + str(depth)}] chunk {chunk} round "
                            f"{round_tokens} x{n_rounds} slots {'all' if n_slots >= 1 << 29 else n_slots}{tier_note}: est "
                            f"{est:.0f} ms (compute {comp:.0f}, pcie {pcie_ms:.0f}, nvlink {nv_ms:.0f})")
                        key = (est, SHARD_MODES.index(mode), -chunk)
                        if best is None or key < best[0]:
                            best = (key, cfg)
                if best is not None and best[1].shard == mode and resid == "all" and best[1].n_gpu_opt_layers is None:
                    break       # fully resident fits: no reason to look at offloaded variants of this mode

    for head_rows in head_rows_options:
        if best is None:
            search(head_rows)
    if best is None:
        need = (P + G + O) / max(dp, 1) + mm.embed_head_resident
        if need > gpu_budget and (P + G + O) > host_budget:
            raise ValueError(
                f"infeasible (host-bound): model states need {(P + G + O) / GiB:.1f} GiB but the host budget is "
                f"{host_budget / GiB:.1f} GiB and the GPU budget {gpu_budget / GiB:.1f} GiB; raise --max-host-mem-gib, "
                f"use LoRA, or add GPUs")
        raise ValueError(
            f"infeasible (GPU-bound): no chunk size in [{lo_chunk}, {hi_chunk}] leaves room for two activation slots "
            f"in {gpu_budget / GiB:.1f} GiB; lower --min-chunk-size or raise --max-gpu-mem-gib")
    cfg = best[1]
    cfg.report = log
    say(f"chosen: shard={cfg.shard} chunk={cfg.max_chunk_size} round={cfg.target_round_tokens} rounds="
        f"{cfg.target_num_rounds} n_gpu_layers={cfg.n_gpu_layers} n_gpu_grads={cfg.n_gpu_grads} "
        f"n_gpu_opt_layers={cfg.n_gpu_opt_layers} est {cfg.est_step_ms:.0f} ms")
    return cfg


def _round_down_to_multiple(tokens: int, chunk: int, batch: int) -> int:
    """Round size: a multiple of the chunk, preferring divisors of the per-rank batch (no short tail round)."""
    tokens = max(chunk, tokens // chunk * chunk)
    if tokens >= batch:
        return batch
    n_rounds = math.ceil(batch / tokens)
    even = math.ceil(batch / n_rounds / chunk) * chunk
    return min(tokens, max(chunk, even))


def _chunk_candidates(batch: int, max_seq_len: int, lo: int, hi: int) -> List[int]:
    """Candidate chunk sizes, largest first: divisors of the batch and powers of two inside [lo, hi]; a chunk
    holds whole sequences whenever ``max_seq_len <= hi``."""
    c = {d for d in divisors(batch) if lo <= d <= hi}
    p = 1
    while p <= hi:
        if p >= lo:
            c.add(p)
        p *= 2
    if max_seq_len <= hi:
        c = {x for x in c if x >= max_seq_len} or {max_seq_len}
    c = c or {min(max(lo, 1), hi)}
    return sorted(c, reverse=True)
