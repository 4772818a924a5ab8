"""Data parallelism over one NVSwitch box with sharded gradients and optimizer state.

Two interchangeable back ends behind the same engine hooks:

``P2PDataParallel`` (the product, CUDA):  parameters and gradients of all ranks live in peer-mapped
arenas.  As soon as a layer's backward has finished on the last accumulation round, a comm stream runs
(1) a flag exchange — "my gradients of layer l are final" — with a bounded wait for all peers, and
(2) the fused reduce-scatter kernel: each rank sums ITS element range of the W gradient buffers straight
out of peer memory, casts bf16→fp32, applies the ``1/tokens`` scale and writes a local fp32 shard.  This
overlaps the backward of layer l-1.  ``step()`` then runs the sharded AdamW kernel, whose store loop
writes the new bf16 parameters into every rank's parameter arena (the all-gather is fused into the
optimizer), and closes with one flag barrier.  No NCCL call is made on this path.

With ``shard="opt+grad+param"`` the parameter all-gather of the large (bf16) segments of attention layers is
deferred: the optimizer writes only the rank's own range, and the FIRST GEMM that consumes the layer's weights in the
next forward (the QKV projection) pulls the other ranks' ranges of the whole layer out of peer memory while it computes
(``ftb_gemm_bf16_wgather``, comm mode 3 of the tcgen05 GEMM), gating each weight tile on the arrival of its bytes.

``CollectiveDataParallel`` (the baseline, any backend incl. gloo on CPU):  ``all_reduce`` of each
layer's gradients, then the ordinary local optimizer on replicated state.

The reference project is single-GPU; its closest analogue is gradient accumulation across rounds
(flextrain/engine/active_model.py:338-411) and a design note proposing ZeRO-1 by layer
(docs/internal/NOTES.md:2340-2385).
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_long, c_uint, c_void_p
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..core.layer import itemsize
from .comm import PeerGroup, shard_range

_DT = {torch.bfloat16: 0, torch.float32: 1}


@dataclass
class Segment:
    """A run of same-dtype, equally treated tensors inside a unit's parameter and gradient buffers."""
    p_off: int          # byte offset in the parameter arena
    g_off: int          # byte offset in the gradient arena
    numel: int
    p_dtype: torch.dtype
    g_dtype: torch.dtype
    decay: bool
    begin: int = 0      # this rank's range
    count: int = 0
    shard_off: int = 0  # element offset in the rank's fp32 shard arrays
    name: Optional[str] = None   # set for a tensor that one rank owns whole (matrix optimizers need the full gradient)
    shape: Tuple[int, ...] = ()
    owner: int = -1


def build_segments(lb, p_base: int, g_base: int, no_decay_1d: bool = True, whole=()) -> List[Segment]:
    """Merge tensors that are adjacent in both buffers and share dtypes / decay into segments.  Tensors named in
    ``whole`` stay segments of their own (they are reduced to, and updated by, a single owner rank)."""
    segs: List[Segment] = []
    for t in lb.spec.trainable():
        if t.is_local_part:
            continue            # owned by this rank alone (expert / tensor parallel part): no reduction, local update
        po, pn, _, pdt = lb.p_layout[t.name]
        go, gn, _, gdt = lb.g_layout[t.grad_name]
        decay = not (no_decay_1d and len(t.shape) == 1)
        s = Segment(p_base + po, g_base + go, t.numel, pdt, gdt, decay)
        if t.name in whole:
            s.name, s.shape = t.name, tuple(t.shape)
            segs.append(s)
            continue
        if segs and segs[-1].name is None:
            q = segs[-1]
            if (q.p_dtype == pdt and q.g_dtype == gdt and q.decay == decay
                    and q.p_off + q.numel * itemsize(pdt) == s.p_off and q.g_off + q.numel * itemsize(gdt) == s.g_off):
                q.numel += t.numel
                continue
        segs.append(s)
    return segs


class _Base:
    def __init__(self, rank: int, world: int, device, process_group=None):
        self.rank, self.world, self.device, self.pg = rank, world, torch.device(device), process_group
        self.am = None
        # hybrid grids: the group of ranks that hold the same tensor- / expert-parallel part, and its first rank
        self.replica_pg, self.replica_src = None, 0

    def attach(self, am) -> None:
        self.am = am

    def buffer_kwargs(self) -> dict:
        return {}

    def after_weights_loaded(self, am) -> None:
        """Make every rank start from rank 0's weights."""
        import torch.distributed as dist
        for scope, l, name, t in am.named_master_params():
            if not am.spec_of(scope, l, name).is_local_part:
                dist.broadcast(t, src=0, group=self.pg)
            elif self.replica_pg is not None:
                dist.broadcast(t, src=self.replica_src, group=self.replica_pg)

    @staticmethod
    def local_part_names(spec) -> List[str]:
        return [t.name for t in spec.trainable() if t.is_local_part]

    def on_layer_grads_ready(self, layer: int) -> None: ...
    def on_embed_head_grads_ready(self) -> None: ...


class CollectiveDataParallel(_Base):
    """Baseline: library all-reduce of every unit's gradient buffer + replicated optimizer."""

    def _allreduce(self, buf: torch.Tensor, lb) -> None:
        import torch.distributed as dist
        part = {t.grad_name for t in lb.spec.trainable() if t.is_local_part}
        for name, (off, nb, shape, dt) in lb.g_layout.items():
            if name not in part:
                dist.all_reduce(buf[off:off + nb].view(dt), group=self.pg)
            elif self.replica_pg is not None:        # the same part on other model-parallel groups saw other data
                dist.all_reduce(buf[off:off + nb].view(dt), group=self.replica_pg)

    def on_layer_grads_ready(self, layer: int) -> None:
        bm = self.am.buffers
        self._allreduce(bm.grad_buffer(layer), bm.layers[layer])

    def on_embed_head_grads_ready(self) -> None:
        bm = self.am.buffers
        self._allreduce(bm.embed_g, bm.embed)
        self._allreduce(bm.head_g, bm.head)

    def step(self, am) -> int:
        return am._step_local()


class P2PDataParallel(_Base):
    def __init__(self, rank: int, world: int, device, process_group=None, timeout_s: float = 60.0):
        super().__init__(rank, world, device, process_group)
        self.group = PeerGroup(rank, world, device, process_group, timeout_s=timeout_s)
        self.lib = self.group.lib
        self.units: Dict[object, List[Segment]] = {}
        self.grad_shard = self.m = self.v = None
        self._reduced_epoch = None

    # ------------------------------------------------------------------- set-up
    def buffer_kwargs(self) -> dict:
        # FTB_DP_MULTIMEM=1: the gradient arena is bound to an NVSwitch multicast object and the reduce-scatter pulls
        # in-switch sums (multimem.ld_reduce) instead of reading every peer's copy
        import os
        mm = os.environ.get("FTB_DP_MULTIMEM", "0") == "1"
        return {"device_alloc": lambda nbytes, tag: self.group.alloc(nbytes, multicast=(mm and tag == "grads")),
                "shard_opt": True}

    def attach(self, am) -> None:
        from ..optim import AdamW, HybridMuonAdamW, Muon, uses_muon
        opt = am.optimizer
        # Element-wise AdamW is sharded by element range.  Muon orthogonalises whole matrices, so each of its tensors is
        # reduced to ONE owner rank (owners balanced by element count), updated there with the tcgen05 Newton-Schulz
        # GEMMs and pushed to the peers' arenas by stores: the step's matrix work is split over the ranks instead of
        # being repeated on each.
        if isinstance(opt, AdamW):
            self.adamw, self.muon, is_muon = opt, None, (lambda t: False)
        elif isinstance(opt, Muon):
            self.adamw, self.muon, is_muon = None, opt, (lambda t: True)
        elif isinstance(opt, HybridMuonAdamW):
            self.adamw, self.muon, is_muon = opt.adamw, opt.muon, uses_muon
        else:
            raise TypeError(f"the peer-memory data-parallel path knows AdamW, Muon and their hybrid, not {type(opt).__name__}")
        self.am = am
        bm = am.buffers
        nd = self.adamw.no_decay_1d if self.adamw is not None else True
        off = 0
        keys = ["embed"] + list(range(len(am.layers))) + ["head"]
        lbs = {"embed": bm.embed, "head": bm.head, **{i: lb for i, lb in enumerate(bm.layers)}}
        load = [0] * self.world
        self.owned_state: Dict[object, Dict[str, torch.Tensor]] = {}     # Muon momentum of the tensors this rank owns
        for key in keys:
            whole = {t.name for t in lbs[key].spec.trainable() if not t.is_local_part and is_muon(t)}
            segs = build_segments(lbs[key], bm.p_off[key], bm.g_off[key], nd, whole)
            for s in segs:
                if s.name is not None:
                    s.owner = min(range(self.world), key=lambda r: (load[r], r))
                    load[s.owner] += s.numel
                    s.begin, s.count = (0, s.numel) if s.owner == self.rank else (0, 0)
                    if s.owner == self.rank:
                        self.owned_state.setdefault(key, {})[s.name] = torch.zeros(
                            s.shape, dtype=self.muon.state_dtype, device=self.device)
                else:
                    s.begin, s.count = shard_range(s.numel, self.rank, self.world)
                s.shard_off = off
                off += (s.count + 7) // 8 * 8
            self.units[key] = segs
        n = max(off, 8)
        f32 = lambda: torch.zeros(n, dtype=torch.float32, device=self.device)
        self.grad_shard, self.m, self.v = f32(), f32(), f32()
        # tensors owned by this rank alone (its slice of every tensor- / expert-parallel matrix) keep an ordinary local
        # optimizer with fp32 state.  When the planner could not fit that state into HBM (``n_gpu_opt_layers`` set: a
        # 70B model over 8 tensor-parallel ranks carries 70 GB of it per rank) it lives in pinned host memory, one
        # flat buffer per unit, and streams through ``opt_ring`` device buffers during ``step()``.
        self.local_names: Dict[object, List[str]] = {}
        self.local_state: Dict[object, Dict[str, torch.Tensor]] = {}
        self.opt_on_host = getattr(am.ws, "n_gpu_opt_layers", None) is not None
        self._state_layout: Dict[object, List] = {}
        self._state_flat: Dict[object, torch.Tensor] = {}
        for key in keys:
            names = self.local_part_names(lbs[key].spec)
            if not names:
                continue
            self.local_names[key] = names
            specs = [s for s in am.optimizer.state_specs(lbs[key].spec) if s.param in names]
            if not self.opt_on_host:
                self.local_state[key] = {s.key: torch.zeros(s.shape, dtype=torch.float32, device=self.device)
                                         for s in specs}
                continue
            lay, n = [], 0
            for s in specs:
                cnt = 1
                for d in s.shape:
                    cnt *= d
                lay.append((s.key, n, cnt, tuple(s.shape)))
                n += (cnt + 63) // 64 * 64
            flat = bm.host.alloc(max(n, 1) * 4).view(torch.float32)
            flat.zero_()
            self._state_layout[key], self._state_flat[key] = lay, flat
            self.local_state[key] = {k2: flat[o:o + c].view(shp) for k2, o, c, shp in lay}    # host views (checkpoints)
        if self.opt_on_host and self._state_flat:
            depth = max(2, int(am.ws.n_gpu_opt_layers))
            biggest = max(f.numel() for f in self._state_flat.values())
            self.opt_ring = [torch.empty(biggest, dtype=torch.float32, device=self.device) for _ in range(depth)]
        # deferred parameter all-gather ("opt+grad+param"): bf16 segments of attention layers are gathered by the
        # layer's first GEMM; everything else (norm weights, embedding, head, other layer kinds) is pushed eagerly
        # (element-range shards only: a matrix optimizer's owner pushes whole tensors right after its update)
        self.defer = getattr(am.ws, "shard", "") == "opt+grad+param" and self.muon is None
        self.deferred_keys = set()
        if self.defer:
            for i, layer in enumerate(am.layers):
                big = [s for s in self.units[i] if s.p_dtype == torch.bfloat16]
                if getattr(layer, "attn", None) is not None and getattr(layer.cfg, "lora", None) is None \
                        and 1 <= len(big) <= 4 and all((s.numel * 2) % 16 == 0 for s in big):
                    self.deferred_keys.add(i)
        self._stale = set()
        self._gather_counter = torch.zeros(8, dtype=torch.int64, device=self.device)
        self.slot = {k: i for i, k in enumerate(keys)}
        self.barrier_slot = len(keys)
        self.comm_stream = am.streams.comm
        self._ev = {}

    # ---------------------------------------------------------------- kernel calls
    def _tables(self, segs: List[Segment], kind: str):
        n = len(segs)
        arr = lambda vals, ct=c_long: (ct * n)(*vals)
        if kind == "grad":
            return n, arr([s.g_off for s in segs]), arr([s.begin for s in segs]), arr([s.count for s in segs]), \
                arr([s.shard_off for s in segs]), arr([_DT[s.g_dtype] for s in segs], c_int)
        return n, arr([s.p_off for s in segs]), arr([s.begin for s in segs]), arr([s.count for s in segs]), \
            arr([s.shard_off for s in segs]), arr([_DT[s.p_dtype] for s in segs], c_int)

    def _reduce_unit(self, key, scale: float, stream) -> None:
        from .. import ops
        segs = self.units[key]
        bm = self.am.buffers
        mc = getattr(bm.grad_arena, "mc_ptr", 0)
        for i0 in range(0, len(segs), 16):
            n, boff, beg, cnt, ooff, dts = self._tables(segs[i0:i0 + 16], "grad")
            if mc:
                rc = self.lib.ftb_comm_reduce_scatter_mc(c_void_p(mc), bm.grad_arena.c_ptrs, c_int(n), boff, beg, cnt,
                                                         ooff, dts, c_void_p(self.grad_shard.data_ptr()),
                                                         c_int(self.world), c_float(scale),
                                                         c_void_p(stream.cuda_stream))
            else:
                rc = self.lib.ftb_comm_reduce_scatter(bm.grad_arena.c_ptrs, c_int(n), boff, beg, cnt, ooff, dts,
                                                      c_void_p(self.grad_shard.data_ptr()), c_int(self.world),
                                                      c_int(self.rank), c_float(scale), c_void_p(stream.cuda_stream))
            if rc != 0:
                raise RuntimeError(f"ftb_comm_reduce_scatter failed ({rc})")
            ops._count()

    def _reduce(self, key) -> None:
        """Flag exchange + fused reduce-scatter of one unit on the comm stream, after compute produced its grads."""
        st = self.am.streams
        cs = self.comm_stream
        ev = torch.cuda.Event()
        ev.record(st.compute)
        cs.wait_event(ev)
        self.group.signal_wait(self.slot[key], self._epoch, cs)
        self._reduce_unit(key, 1.0, cs)

    def _call_epoch(self) -> None:
        """One flag epoch per ``fwd_bwd`` call, not per optimizer step.  Gradients may be accumulated over several
        calls before ``step()``; every call re-reduces the accumulated buffers (the shard is overwritten, so the last
        call's sum is the one the optimizer sees).  With a single epoch per step the later calls would find the flags
        of the first call already raised, skip the wait and sum peers' buffers that are still being accumulated.
        Every rank must make the same number of ``fwd_bwd`` calls per step."""
        serial = (self.am.step_num, getattr(self.am, "fwd_bwd_serial", 0))
        if self._reduced_epoch != serial:
            self._epoch = self.group.next_epoch()
            self._reduced_epoch = serial

    def on_layer_grads_ready(self, layer: int) -> None:
        self._call_epoch()
        self._reduce(layer)

    def on_embed_head_grads_ready(self) -> None:
        self._call_epoch()
        self._reduce("embed")
        self._reduce("head")

    def grad_norm(self, am) -> float:
        """Global L2 norm of the reduced gradient, from the shards: every rank squares its own fp32 range of each
        replicated tensor (the alignment padding between ranges is never written and stays zero) plus its own slices
        of tensor- / expert-parallel tensors, and one scalar all-reduce adds them up (one host read)."""
        import torch.distributed as dist
        cs = self.comm_stream
        cs.wait_stream(am.streams.compute)
        with torch.cuda.stream(cs):
            sq = self.grad_shard.pow(2).sum()
            for key, names in self.local_names.items():
                bm = am.buffers
                spec, grads = {"embed": (bm.embed.spec, bm.embed_grads()), "head": (bm.head.spec, bm.head_grads())}.get(
                    key) or (bm.layers[key].spec, bm.grads(key))
                for t in spec.trainable():
                    if t.name in names and grads.get(t.grad_name) is not None:
                        sq = sq + grads[t.grad_name].to(torch.float32).pow(2).sum()
            dist.all_reduce(sq, group=self.pg)
            out = float(sq.sqrt())
        return out

    def step(self, am, grad_scale: float = 1.0) -> int:
        from .. import ops
        opt = am.optimizer
        cs = self.comm_stream
        bm = am.buffers
        step = am.step_num
        if grad_scale != 1.0:                   # clipping: the reduced fp32 shard is what the sharded AdamW reads
            with torch.cuda.stream(cs):
                self.grad_shard.mul_(grad_scale)
        ad = self.adamw
        if ad is not None:
            bc1, bc2 = 1.0 - ad.beta1 ** step, 1.0 - ad.beta2 ** step
        own_only = (c_void_p * 1)(bm.param_arena.c_ptrs[self.rank])       # a one-rank "group": no peer stores
        for key, segs in self.units.items():
            deferred = key in self.deferred_keys
            elem = [s for s in segs if s.name is None]
            groups = [([s for s in elem if not (deferred and s.p_dtype == torch.bfloat16)], False),
                      ([s for s in elem if deferred and s.p_dtype == torch.bfloat16], True)]
            for glist, local in groups:
                for i0 in range(0, len(glist), 16):
                    part = glist[i0:i0 + 16]
                    n, boff, beg, cnt, ooff, dts = self._tables(part, "param")
                    mask = sum((1 << i) for i, s in enumerate(part) if s.decay)
                    rc = self.lib.ftb_comm_adamw_push(own_only if local else bm.param_arena.c_ptrs, c_int(n), boff, beg,
                                                      cnt, ooff, dts, c_void_p(self.grad_shard.data_ptr()),
                                                      c_void_p(self.m.data_ptr()), c_void_p(self.v.data_ptr()),
                                                      c_int(1 if local else self.world), c_int(0 if local else self.rank),
                                                      c_float(ad.lr), c_float(ad.beta1), c_float(ad.beta2),
                                                      c_float(ad.eps), c_float(ad.weight_decay), c_float(bc1),
                                                      c_float(bc2), c_uint(mask), c_void_p(cs.cuda_stream))
                    if rc != 0:
                        raise RuntimeError(f"ftb_comm_adamw_push failed ({rc})")
                    ops._count()
            if deferred:
                self._stale.add(key)
            mine = [s for s in segs if s.name is not None and s.owner == self.rank]
            if mine:
                mu = self.muon
                pv = bm.embed_params() if key == "embed" else bm.head_params() if key == "head" else bm.params(key)
                with torch.cuda.stream(cs):
                    for s in mine:
                        g = self.grad_shard[s.shard_off:s.shard_off + s.numel].view(s.shape)      # fp32, fully reduced
                        ops.muon_step(pv[s.name], g, self.owned_state[key][s.name], lr=mu.lr, beta=mu.beta,
                                      weight_decay=mu.weight_decay, ns_iters=mu.ns_iters, nesterov=mu.nesterov)
                        nbytes = (s.numel * itemsize(s.p_dtype) + 15) // 16 * 16     # layout slots are padded past this
                        rc = self.lib.ftb_comm_allgather_push(bm.param_arena.c_ptrs, c_long(s.p_off), c_long(nbytes),
                                                              c_int(self.world), c_int(self.rank),
                                                              c_void_p(cs.cuda_stream))
                        if rc != 0:
                            raise RuntimeError(f"ftb_comm_allgather_push failed ({rc})")
                        ops._count()
        if self.local_names and self.opt_on_host:
            self._step_local_streamed(am, opt, step, grad_scale)
        elif self.local_names:
            cs.wait_stream(am.streams.compute)
            with torch.cuda.stream(cs):
                for key, names in self.local_names.items():
                    opt.step(bm.layers[key].spec, bm.params(key), bm.grads(key), self.local_state[key], step,
                             grad_scale, only=set(names))
        # every peer's stores into my parameters have landed, and every peer is done reading my gradients
        self.group.signal_wait(self.barrier_slot, self.group.next_epoch(), cs)
        am.streams.compute.wait_stream(cs)
        return 0

    def _step_local_streamed(self, am, opt, step: int, grad_scale: float = 1.0) -> None:
        """Update this rank's own slices with their optimizer state streaming through the host: unit k's state is
        copied into ring slot ``k % depth`` on the inbound stream while unit k-1 is updated on the comm stream and
        unit k-2 is written back on the outbound stream (one coalesced copy per unit and direction; the single-GPU
        pattern of flextrain/engine/active_model.py:428-658 applied to a model-parallel rank)."""
        st, bm, cs = am.streams, am.buffers, self.comm_stream
        keys = list(self.local_names)
        depth = len(self.opt_ring)
        cs.wait_stream(st.compute)
        st.inbound.wait_stream(st.compute)
        loaded = [torch.cuda.Event() for _ in keys]
        updated = [torch.cuda.Event() for _ in keys]
        stored = [torch.cuda.Event() for _ in keys]

        def fetch(i: int) -> None:
            flat = self._state_flat[keys[i]]
            with torch.cuda.stream(st.inbound):
                if i >= depth:
                    st.inbound.wait_event(stored[i - depth])          # the slot's previous tenant is back on the host
                self.opt_ring[i % depth][: flat.numel()].copy_(flat, non_blocking=True)
                loaded[i].record(st.inbound)

        for i in range(min(depth - 1, len(keys))):
            fetch(i)
        for i, key in enumerate(keys):
            if i + depth - 1 < len(keys):
                fetch(i + depth - 1)
            dev = self.opt_ring[i % depth]
            views = {k2: dev[o:o + c].view(shp) for k2, o, c, shp in self._state_layout[key]}
            cs.wait_event(loaded[i])
            with torch.cuda.stream(cs):
                opt.step(bm.layers[key].spec, bm.params(key), bm.grads(key), views, step, grad_scale,
                         only=set(self.local_names[key]))
                updated[i].record(cs)
            with torch.cuda.stream(st.outbound):
                st.outbound.wait_event(updated[i])
                flat = self._state_flat[key]
                flat.copy_(dev[: flat.numel()], non_blocking=True)
                stored[i].record(st.outbound)
        cs.wait_stream(st.outbound)

    def first_gemm(self, layer: int, x: torch.Tensor, w: torch.Tensor):
        """``x @ w.T`` for the first projection of ``layer`` in a step, fused with the all-gather of the layer's
        deferred parameter segments (peer pulls inside the GEMM kernel).  Returns ``None`` when the layer's parameters
        are already current (later rounds of the step, recompute, layers that are pushed eagerly)."""
        if layer not in self._stale:
            return None
        from .. import ops
        from ..ops.cuda import load, _stream
        bm = self.am.buffers
        segs = [s for s in self.units[layer] if s.p_dtype == torch.bfloat16]
        base = bm.param_arena.ptrs[self.rank]
        rel = w.data_ptr() - base
        first = [s for s in segs if s.p_off <= rel and rel + w.numel() * 2 <= s.p_off + s.numel * 2]
        if not first or x.dtype != torch.bfloat16 or not w.is_contiguous() or x.stride(1) != 1:
            raise RuntimeError("deferred parameter gather: the first projection's weight is not inside one bf16 segment")
        order = first + [s for s in segs if s is not first[0]]
        n = len(order)
        W = self.world
        per = lambda s: (s.numel + 8 * W - 1) // (8 * W) * 8
        arr = lambda vals, ct=c_long: (ct * n)(*vals)
        self._gather_counter.zero_()
        M, K = x.shape
        N = w.shape[0]
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        rc = load("gemm_tcgen05").ftb_gemm_bf16_wgather(
            c_void_p(x.data_ptr()), c_void_p(w.data_ptr()), c_void_p(out.data_ptr()), c_int(M), c_int(N), c_int(K),
            c_int(x.stride(0)), c_int(N), c_float(1.0), bm.param_arena.c_ptrs, c_int(n),
            arr([s.p_off for s in order]), arr([s.numel for s in order]), arr([2] * n, c_int),
            arr([per(s) for s in order]), c_void_p(self._gather_counter.data_ptr()), c_int(W), c_int(self.rank),
            c_int(0), _stream())
        if rc != 0:
            raise RuntimeError(f"ftb_gemm_bf16_wgather failed ({rc})")
        ops._count()
        self._stale.discard(layer)
        return out

    def finish_param_gather(self) -> None:
        """Complete the deferred all-gather of every layer that has not run a forward since the last optimizer step
        (before exporting, evaluating a single rank's copy, or comparing ranks): each rank pushes its own ranges."""
        if not self._stale:
            return
        bm = self.am.buffers
        cs = self.comm_stream
        cs.wait_stream(self.am.streams.compute)
        for key in sorted(self._stale):
            for s in self.units[key]:
                if s.p_dtype != torch.bfloat16 or s.count == 0:
                    continue
                rc = self.lib.ftb_comm_allgather_push(bm.param_arena.c_ptrs, c_long(s.p_off + s.begin * 2),
                                                      c_long(s.count * 2), c_int(self.world), c_int(self.rank),
                                                      c_void_p(cs.cuda_stream))
                if rc != 0:
                    raise RuntimeError(f"ftb_comm_allgather_push failed ({rc})")
        self.group.signal_wait(self.barrier_slot, self.group.next_epoch(), cs)
        self.am.streams.compute.wait_stream(cs)
        self._stale.clear()

    def check(self) -> None:
        self.group.check()


def emulate_sharded_step(grad_bufs: List[torch.Tensor], param_bufs: List[torch.Tensor], segs_per_rank, states, *,
                         lr, beta1, beta2, eps, wd, step: int, scale: float = 1.0) -> None:
    """Single-process statement of what the two kernels do over ``W`` ranks' buffers (CPU test oracle):
    rank r reduces its ranges of all ``grad_bufs`` and writes the AdamW result into all ``param_bufs``."""
    W = len(grad_bufs)
    bc1, bc2 = 1.0 - beta1 ** step, 1.0 - beta2 ** step
    for r in range(W):
        m, v = states[r]
        for s in segs_per_rank[r]:
            if s.count == 0:
                continue
            gsz, psz = itemsize(s.g_dtype), itemsize(s.p_dtype)
            g = sum(gb[s.g_off: s.g_off + s.numel * gsz].view(s.g_dtype)[s.begin:s.begin + s.count].to(torch.float32)
                    for gb in grad_bufs) * scale
            pv = param_bufs[r][s.p_off: s.p_off + s.numel * psz].view(s.p_dtype)[s.begin:s.begin + s.count]
            p = pv.to(torch.float32)
            sl = slice(s.shard_off, s.shard_off + s.count)
            p = p - lr * (wd if s.decay else 0.0) * p
            m[sl] = beta1 * m[sl] + (1 - beta1) * g
            v[sl] = beta2 * v[sl] + (1 - beta2) * g * g
            p = p - lr * (m[sl] / bc1) / ((v[sl] / bc2).sqrt() + eps)
            for pb in param_bufs:
                pb[s.p_off: s.p_off + s.numel * psz].view(s.p_dtype)[s.begin:s.begin + s.count] = p.to(s.p_dtype)
