"""Expert parallelism: experts sharded over the ranks of one NVSwitch box, tokens stay data-parallel.

Per MoE layer and chunk, on every rank (all index math on the device, no host sync):

1. route local tokens, sort the ``T*K`` slots by expert, count per expert;
2. all-gather the ``(W, E)`` count table (peer stores + flag exchange) — every rank can now compute, for each of
   its slots, the owning rank and the exact row inside that owner's expert-major receive buffer;
3. **dispatch**: ``ftb_ep_push_rows`` stores each slot's activation row straight into the owner's buffer;
4. owners run the grouped tcgen05 GEMMs (up + GLU + down) over their local experts;
5. **combine**: ``ftb_ep_combine_pull`` reads each slot's result row back from its owner, applies the router weight,
   sums over K and adds the residual.

Backward re-dispatches ``h`` and ``dy`` (with the router weights as a per-row scalar), runs the expert backward and
the per-expert weight gradients on the owner, and combines ``dx`` and the router-weight gradients back.
``backend="collective"`` implements the same contract with all_gather (CPU tests, library baseline).
The reference project has no expert parallelism; its single-GPU MoE path is flextrain/ops/full_moe.py:177-466.
"""
from __future__ import annotations

import os
from ctypes import c_int, c_long, c_void_p
from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops

PAD = 128
FILLER_TOKENS = 128     # length of the unscored chunk a rank runs when its peers have more chunks than it has


def _dist_ready() -> bool:
    import torch.distributed as dist
    return dist.is_available() and dist.is_initialized()

# Receive-buffer capacity as a multiple of the balanced share.  0 (default) = dropless: the buffers hold the worst
# case (every slot of every rank routed to one rank), so no routing skew can overflow them.  Saved activations are
# sized by the rows a rank actually receives, not by this bound.
DEFAULT_CAPACITY_FACTOR = float(os.environ.get("FTB_EP_CAPACITY", "0"))
PLANNING_FACTOR = 1.25          # what the planner assumes a rank receives, relative to the balanced share


def ep_capacity(T: int, K: int, E: int, world: int, factor: float) -> int:
    """Rows of one rank's expert-major receive buffer for chunks of ``T`` tokens per rank: ``factor`` times the
    balanced share ``T*K`` plus tile padding per local expert.  Exceeding it is reported, never written past."""
    if factor <= 0:
        factor = float(world)
    rows = int(min(factor, float(world)) * T * K) + (E // world) * (PAD - 1)
    return (rows + PAD - 1) // PAD * PAD


@dataclass
class EPPlan:
    order: torch.Tensor          # (n,) sorted position -> local slot id
    src_tok: torch.Tensor        # (n,) int32 token of each sorted slot
    dest_rank: torch.Tensor      # (n,) int32
    dest_row: torch.Tensor       # (n,) int32
    slot_rank: torch.Tensor      # (T, K) int32
    slot_row: torch.Tensor       # (T, K) int32
    offsets: torch.Tensor        # (E_local + 1,) int32 rows of my experts (padded segments), clamped to the capacity
    w_sorted: torch.Tensor       # (n,) fp32 router weight of each sorted slot
    rows: int = 0                # padded rows this rank received (host value: one device read per plan)


class ExpertParallel:
    def __init__(self, rank: int, world: int, device, process_group=None, backend: str = "p2p", group=None,
                 capacity_factor: float = DEFAULT_CAPACITY_FACTOR):
        self.rank, self.world, self.device, self.pg, self.backend = rank, world, torch.device(device), process_group, backend
        self.capacity_factor = capacity_factor
        self.group = group
        if backend == "p2p":
            from ..ops.cuda import load
            if group is None:
                from .comm import PeerGroup
                self.group = PeerGroup(rank, world, device, process_group)
            self.lib = load("moe")
        self._bufs = {}
        self._calls = 0
        self.slot_base = 3500
        self.overflow = None
        self._overflow_dev = None
        self.max_chunk_tokens = 0      # set by attach(): the planner's chunk size, identical on every rank

    def attach(self, am) -> None:
        """Bind to the engine.  Receive / result / scalar buffers are symmetric allocations (every rank must ask for
        the same size in the same order), and the library gathers need equal shapes, so their size comes from the
        planner's ``max_chunk_size`` (the same number on every rank) and not from the token count of the chunk at
        hand: data-parallel ranks read different sequences and their chunks differ in length."""
        self.max_chunk_tokens = int(am.ws.max_chunk_size)

    # ------------------------------------------------------------------ helpers
    def capacity(self, T: int, K: int, E: int) -> int:
        return ep_capacity(max(T, self.max_chunk_tokens), K, E, self.world, self.capacity_factor)

    def agree_max(self, n: int) -> int:
        """Largest ``n`` over the ranks (one small all-reduce, a host read).  Every MoE layer does flag exchanges and
        peer reads per chunk, so the ranks of an expert-parallel group must walk the same number of rounds and of
        chunks per round; the engine pads the shorter ranks with filler chunks up to this count."""
        if self.world <= 1 or self.pg is None and not _dist_ready():
            return n
        import torch.distributed as dist
        t = torch.tensor([n], dtype=torch.int64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.pg)
        return int(t.item())

    def _sync(self) -> None:
        if self.backend == "p2p":
            self.group.signal_wait(self.slot_base + (self._calls % 64), self.group.next_epoch())
            self._calls += 1

    def _buf(self, name: str, nbytes: int):
        key = (name, nbytes)
        if key not in self._bufs:
            self._bufs[key] = self.group.alloc(nbytes)
        return self._bufs[key]

    def _gather_counts(self, counts: torch.Tensor, as_int32: bool = False) -> torch.Tensor:
        W, E = self.world, counts.numel()
        if self.backend != "p2p":
            import torch.distributed as dist
            table = torch.empty(W * E, dtype=counts.dtype, device=counts.device)
            dist.all_gather_into_tensor(table, counts.contiguous(), group=self.pg)
            return table.view(W, E)
        buf = self._buf("cnt", W * E * 4)
        table = buf.local.view(torch.int32)[: W * E].view(W, E)
        table[self.rank].copy_(counts.to(torch.int32))
        self._sync()                       # everyone's previous readers are done, my row is written
        from ..ops.cuda import _stream
        rc = self.group.lib.ftb_comm_allgather_push(buf.c_ptrs, c_long(self.rank * E * 4), c_long(E * 4),
                                                    c_int(W), c_int(self.rank), _stream())
        if rc != 0:
            raise RuntimeError(f"ftb_comm_allgather_push failed ({rc})")
        self._sync()
        return table.clone() if as_int32 else table.clone().long()

    def plan(self, idx: torch.Tensor, w: torch.Tensor, E: int) -> EPPlan:
        if self.backend == "p2p" and idx.is_cuda and E <= 1024:
            return self._plan_device(idx, w, E)
        T, K = idx.shape
        dev = idx.device
        flat = idx.reshape(-1).long()
        n = flat.numel()
        counts = torch.zeros(E, dtype=torch.long, device=dev).index_add_(0, flat, torch.ones(n, dtype=torch.long, device=dev))
        table = self._gather_counts(counts).long()                      # (W, E)
        return self.plan_from_table(idx, w, E, table)

    def _plan_device(self, idx: torch.Tensor, w: torch.Tensor, E: int) -> EPPlan:
        """The plan on the device: count kernel -> all-gather of the count table over peer memory -> scan + map
        kernels (``csrc/moe.cu``).  No library sort and no eager index arithmetic; the only host read left is the
        row total of the dropless mode (capacity-factor buffers need none: saved activations take the capacity)."""
        from ..ops import cuda as k
        T, K = idx.shape
        counts, work, ex = k.ep_plan_count(idx, E)
        table = self._gather_counts(counts, as_int32=True)
        cap = self.capacity(T, K, E)
        if self._overflow_dev is None:
            self._overflow_dev = torch.zeros((), dtype=torch.int32, device=idx.device)
        slot_rank, slot_row, offsets = k.ep_plan_map(ex, (T, K), E, table, self.world, self.rank, PAD, cap, work,
                                                     self._overflow_dev)
        ops._count(4)
        self.overflow = self._overflow_dev
        rows = cap if self.capacity_factor > 0 else int(offsets[-1])
        return EPPlan(None, None, None, None, slot_rank, slot_row, offsets,
                      w.reshape(-1).to(torch.float32).contiguous(), rows)

    def plan_from_table(self, idx: torch.Tensor, w: torch.Tensor, E: int, table: torch.Tensor) -> EPPlan:
        """The same plan in plain tensor ops (library back end, CPU ranks, and the oracle of the plan kernels):
        ``table (W, E)`` holds every rank's per-expert slot counts."""
        T, K = idx.shape
        dev = idx.device
        W, El = self.world, E // self.world
        flat = idx.reshape(-1).long()
        n = flat.numel()
        order = torch.sort(flat, stable=True).indices
        e_sorted = flat[order]
        counts = table[self.rank]
        tot = table.sum(0)
        padded = (tot + PAD - 1) // PAD * PAD
        pr = padded.view(W, El)
        base = (torch.cumsum(pr, 1) - pr).reshape(E)
        before = torch.cumsum(table, 0) - table
        start_mine = base + before[self.rank]
        src_start = torch.cumsum(counts, 0) - counts
        rank_in = torch.arange(n, device=dev) - src_start[e_sorted]
        dest_rank = (e_sorted // El).to(torch.int32)
        dest_row = (start_mine[e_sorted] + rank_in).to(torch.int32)
        offsets = torch.zeros(El + 1, dtype=torch.int32, device=dev)
        offsets[1:] = torch.cumsum(pr[self.rank], 0).to(torch.int32)
        slot_rank = torch.empty(n, dtype=torch.int32, device=dev)
        slot_row = torch.empty(n, dtype=torch.int32, device=dev)
        slot_rank[order] = dest_rank
        slot_row[order] = dest_row
        cap = self.capacity(T, K, E)
        over = (dest_row >= cap).any()
        self.overflow = over if self.overflow is None else (self.overflow | over)
        # rows past the capacity are never written (the push skips them); the expert GEMMs must not touch them either
        offsets.clamp_(max=cap)
        rows = int(offsets[-1])             # host read: sizes this layer's expert activations by what really arrived
        return EPPlan(order, (order // K).to(torch.int32), dest_rank, dest_row, slot_rank.view(T, K),
                      slot_row.view(T, K), offsets, w.reshape(-1).to(torch.float32)[order].contiguous(), rows)

    # ------------------------------------------------------------- dispatch / combine
    def dispatch(self, x: torch.Tensor, plan: EPPlan, cap: int, name: str, with_scalar: bool = False):
        """Rows of ``x (T, D)`` to their owners. Returns ``(recv (cap, D), recv_scalar (cap,) or None)`` on this rank."""
        T, D = x.shape
        if self.backend != "p2p":
            import torch.distributed as dist
            W = self.world
            rows = x[plan.src_tok.long()].contiguous()
            n = torch.tensor([rows.shape[0]], device=x.device)
            ns = [torch.zeros_like(n) for _ in range(W)]
            dist.all_gather(ns, n, group=self.pg)
            nmax = int(max(int(v) for v in ns))
            pad = lambda t, fill=0: torch.cat([t, torch.full((nmax - t.shape[0], *t.shape[1:]), fill, dtype=t.dtype, device=t.device)])
            def ag(t):
                out = [torch.empty_like(t) for _ in range(W)]
                dist.all_gather(out, t.contiguous(), group=self.pg)
                return torch.cat(out)
            R, DR, DW = ag(pad(rows)), ag(pad(plan.dest_rank, -1)), ag(pad(plan.dest_row))
            S = ag(pad(plan.w_sorted)) if with_scalar else None
            mine = DR == self.rank
            recv = torch.zeros(cap, D, dtype=x.dtype, device=x.device)
            recv[DW[mine].long()] = R[mine]
            sc = None
            if with_scalar:
                sc = torch.zeros(cap, dtype=torch.float32, device=x.device)
                sc[DW[mine].long()] = S[mine]
            return recv, sc
        buf = self._buf(name, cap * D * 2)
        recv = buf.local.view(torch.bfloat16)[: cap * D].view(cap, D)
        R = max(plan.rows, PAD)
        recv[:R].zero_()                   # padding rows inside the used range must read as zero; the rest is never read
        sbuf = sc = None
        if with_scalar:
            sbuf = self._buf(name + "_s", cap * 4)
            sc = sbuf.local.view(torch.float32)[:cap]
            sc[:R].zero_()
        self._sync()                       # all receive buffers are clean and no one still reads the old contents
        from ..ops.cuda import _stream
        if plan.src_tok is None:           # device-built plan: dispatch by (token, k) slot
            Tn, K = plan.slot_rank.shape
            rc = self.lib.ftb_ep_push_slots(c_void_p(x.data_ptr()), c_void_p(plan.slot_rank.data_ptr()),
                                            c_void_p(plan.slot_row.data_ptr()),
                                            c_void_p(plan.w_sorted.data_ptr() if with_scalar else 0), buf.c_ptrs,
                                            sbuf.c_ptrs if with_scalar else None, c_long(Tn * K), c_int(K), c_int(D),
                                            c_long(cap), c_int(self.world), _stream())
        else:
            n = plan.src_tok.numel()
            rc = self.lib.ftb_ep_push_rows(c_void_p(x.data_ptr()), c_void_p(plan.src_tok.data_ptr()),
                                           c_void_p(plan.dest_rank.data_ptr()), c_void_p(plan.dest_row.data_ptr()),
                                           c_void_p(plan.w_sorted.data_ptr() if with_scalar else 0), buf.c_ptrs,
                                           sbuf.c_ptrs if with_scalar else None, c_long(n), c_int(D), c_long(cap),
                                           c_int(self.world), _stream())
        if rc != 0:
            raise RuntimeError(f"ftb_ep dispatch failed ({rc})")
        ops._count()
        self._sync()                       # every rank's rows have landed
        return recv, sc

    def combine(self, y: torch.Tensor, plan: EPPlan, w: Optional[torch.Tensor], resid: Optional[torch.Tensor], cap: int,
                name: str) -> torch.Tensor:
        """``out[t] = resid[t] + sum_k w[t,k] * Y_owner[row(t,k)]``; ``y (cap, D)`` is this rank's expert output."""
        T, K = plan.slot_rank.shape
        D = y.shape[1]
        if self.backend != "p2p":
            import torch.distributed as dist
            if y.shape[0] < cap:            # ranks receive different row counts; the library gather wants equal shapes
                y = torch.cat([y, y.new_zeros(cap - y.shape[0], D)])
            ys = [torch.empty_like(y) for _ in range(self.world)]
            dist.all_gather(ys, y.contiguous(), group=self.pg)
            Y = torch.stack(ys)                                           # (W, cap, D)
            g = Y[plan.slot_rank.long(), plan.slot_row.long()].to(torch.float32)
            if w is not None:
                g = g * w.unsqueeze(-1)
            out = g.sum(1)
            if resid is not None:
                out = out + resid.to(torch.float32)
            return out.to(y.dtype)
        buf = self._buf(name, cap * D * 2)
        ysym = buf.local.view(torch.bfloat16)[: cap * D].view(cap, D)
        if ysym.data_ptr() != y.data_ptr():
            ysym[: y.shape[0]].copy_(y)
        self._sync()                       # all owners' outputs are complete
        out = torch.empty(T, D, dtype=torch.bfloat16, device=y.device)
        from ..ops.cuda import _stream
        rc = self.lib.ftb_ep_combine_pull(buf.c_ptrs, c_void_p(plan.slot_rank.data_ptr()),
                                          c_void_p(plan.slot_row.data_ptr()),
                                          c_void_p(w.contiguous().data_ptr() if w is not None else 0),
                                          c_void_p(resid.data_ptr() if resid is not None else 0),
                                          c_void_p(out.data_ptr()), c_int(T), c_int(K), c_int(D), c_long(cap),
                                          c_int(self.world), _stream())
        if rc != 0:
            raise RuntimeError(f"ftb_ep_combine_pull failed ({rc})")
        ops._count()
        return out

    def pull_scalar(self, v: torch.Tensor, plan: EPPlan, cap: int, name: str) -> torch.Tensor:
        """Per-slot scalar read back from the owners: returns ``(T, K)`` fp32."""
        T, K = plan.slot_rank.shape
        if self.backend != "p2p":
            import torch.distributed as dist
            if v.shape[0] < cap:
                v = torch.cat([v, v.new_zeros(cap - v.shape[0])])
            vs = [torch.empty_like(v) for _ in range(self.world)]
            dist.all_gather(vs, v.contiguous(), group=self.pg)
            return torch.stack(vs)[plan.slot_rank.long(), plan.slot_row.long()]
        buf = self._buf(name, cap * 4)
        vsym = buf.local.view(torch.float32)[:cap]
        vsym[: v.shape[0]].copy_(v)
        self._sync()
        out = torch.empty(T, K, dtype=torch.float32, device=v.device)
        from ..ops.cuda import _stream
        rc = self.lib.ftb_ep_pull_scalar(buf.c_ptrs, c_void_p(plan.slot_rank.data_ptr()),
                                         c_void_p(plan.slot_row.data_ptr()), c_void_p(out.data_ptr()), c_long(T * K),
                                         c_long(cap), c_int(self.world), _stream())
        if rc != 0:
            raise RuntimeError(f"ftb_ep_pull_scalar failed ({rc})")
        return out

    # ------------------------------------------------------------------ MoE layer hooks
    def moe_forward(self, moe, h, x_resid, w, idx, params, slot):
        c = moe.cfg
        F, T = c.expert_dim, h.shape[0]
        cap = self.capacity(T, c.top_k, c.num_experts)
        plan = self.plan(idx, w, c.num_experts)
        xs, _ = self.dispatch(h, plan, cap, "recv_a")
        R = max(plan.rows, PAD)
        up = ops.grouped_gemm(xs[:R], moe.weight(params, "w_up"), plan.offsets)
        slot._t["x_up"] = up               # sized by the rows that arrived, not by the receive capacity
        slot._t["_ep_plan"] = plan
        act = ops.glu_fwd(up[:, F:], up[:, :F], c.kind)
        y = ops.grouped_gemm(act, moe.weight(params, "w_down"), plan.offsets)
        return self.combine(y, plan, w, x_resid, cap, "ybuf")

    def moe_backward(self, moe, dx, h, w, idx, params, grads, slot):
        c = moe.cfg
        F, T, K = c.expert_dim, h.shape[0], c.top_k
        cap = self.capacity(T, K, c.num_experts)
        plan = slot._t.get("_ep_plan") or self.plan(idx, w, c.num_experts)
        R = max(plan.rows, PAD)
        xs, _ = self.dispatch(h, plan, cap, "recv_a")
        dy_u, wrow = self.dispatch(dx, plan, cap, "recv_b", with_scalar=True)
        xs, dy_u, wrow = xs[:R], dy_u[:R], wrow[:R]
        up = slot._t.get("x_up")
        if up is None:
            up = ops.grouped_gemm(xs, moe.weight(params, "w_up"), plan.offsets)
        dact_u = ops.grouped_gemm(dy_u, moe.weight(params, "w_down"), plan.offsets, trans_w=False)
        dup = torch.empty_like(up)
        act_w, dw_rows = ops.glu_bwd_weighted(dact_u, up[:, F:], up[:, :F], wrow, c.kind, dgate=dup[:, F:],
                                              dup=dup[:, :F])
        if "g_down" in grads:           # g_down += dy^T (w * act): the router weight rides on the activation
            ops.grouped_wgrad(dy_u, act_w, plan.offsets, grads["g_down"], pad=PAD)
        if "g_up" in grads:
            ops.grouped_wgrad(dup, xs, plan.offsets, grads["g_up"], pad=PAD)
        moe.lora_wgrad("w_down", dy_u, act_w, plan.offsets, params, grads, PAD)
        moe.lora_wgrad("w_up", dup, xs, plan.offsets, params, grads, PAD)
        dxs = ops.grouped_gemm(dup, moe.weight(params, "w_up"), plan.offsets, trans_w=False)
        dh = self.combine(dxs, plan, None, None, cap, "ybuf")
        dw = self.pull_scalar(dw_rows, plan, cap, "dwbuf")
        return dh, dw

    def check(self) -> None:
        if self.overflow is not None and bool(self.overflow):
            self.overflow = None
            if self._overflow_dev is not None:
                self._overflow_dev.zero_()
            raise RuntimeError("expert-parallel receive capacity exceeded; raise capacity_factor")
        if self.backend == "p2p":
            self.group.check()
