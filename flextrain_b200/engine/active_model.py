"""ActiveModel: the training engine (flextrain/engine/active_model.py:138-2198).

``fwd_bwd(seqs)``: split into rounds → per round pack chunks, plan save levels, then
forward ``for layer: for chunk``, fused head forward+loss+backward per chunk, backward
``for layer↓: for group↓: for chunk↓`` with recompute of the tiers that were not saved, embedding
backward.  ``step()``: optimizer per layer.  No autograd graph exists anywhere.

What differs from the reference, by design for an 8×B200 NVSwitch box:
* state classes are GPU-resident by default; rings over pinned host memory are used only when the
  planner says HBM is too small (n_gpu_layers / n_gpu_grads / n_gpu_opt_layers < n_layers);
* loss bookkeeping stays on the device and is read once per ``fwd_bwd`` (the reference does a
  blocking ``.item()`` per chunk, active_model.py:1307-1313);
* a data-parallel hook fires as soon as a layer's gradients are final, so the fused
  reduce-scatter of layer ``l`` overlaps the backward of layer ``l-1``.
"""
from __future__ import annotations

import ctypes
import dataclasses

import contextlib
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence as Seq

import torch

from ..core.activation_schema import ON_DEVICE, ActivationSlot, fetch_home, send_home
from ..core.layer import ChunkMeta, LayerContext
from ..core.save_level import (HardwareCost, SaveLevelPlan, TransmissionScheduler, build_dp_tables,
                               plan_from_solution)
from ..core.working_set import WorkingSetConfig
from ..io.sequence import Sequence, as_sequence
from .buffers import BufferManager
from .schedule import ChunkPolicy, prepare_training_chunks, split_sequences
from .streams import EventBook, StreamBundle


@dataclass
class StepStats:
    """What one ``fwd_bwd`` did (flextrain/engine/active_model.py:97-129)."""
    loss_sum: float = 0.0
    tokens: int = 0
    active_tokens: int = 0
    n_rounds: int = 0
    n_chunks: int = 0
    fwd_flops: float = 0.0
    recompute_flops: float = 0.0
    attn_fwd_flops: float = 0.0
    host_act_bytes: int = 0
    plan_hist: Dict[int, int] = field(default_factory=dict)
    elapsed_s: float = 0.0

    @property
    def loss(self) -> float:
        return self.loss_sum / max(self.active_tokens, 1)

    # the reference's field names (flextrain/engine/active_model.py:125-129)
    @property
    def total_loss(self) -> float:
        return self.loss_sum

    @property
    def total_tokens(self) -> int:
        return self.tokens

    @property
    def rounds(self) -> int:
        return self.n_rounds


def _nvtx(name: str):
    if torch.cuda.is_available():
        return torch.cuda.nvtx.range(name)
    return contextlib.nullcontext()


class ActiveModel:
    def __init__(self, *, embed, layers, head, optimizer, ws: WorkingSetConfig, device, hw_cost: HardwareCost = None,
                 host_backend=None, dims: Optional[dict] = None, arch: str = "llama", hf_config: Optional[dict] = None,
                 force_saved_act_level: Optional[int] = None, verbose: bool = False, dp=None, tp=None, ep=None,
                 model_dir: Optional[str] = None):
        self.embed, self.layers, self.head = embed, list(layers), head
        self.optimizer = optimizer
        self.ws = ws
        self.device = torch.device(device)
        self.hw = hw_cost or HardwareCost()
        self.dims, self.arch, self.hf_config, self.model_dir = dims or {}, arch, hf_config, model_dir
        self.force_level = force_saved_act_level
        self.verbose = verbose
        self.dp, self.tp, self.ep = dp, tp, ep
        for layer in self.layers:
            if tp is not None:
                layer.bind_tp(tp)
        self.step_num = 0
        self.fwd_bwd_serial = 0          # counts training ``fwd_bwd`` calls (data-parallel flag epochs key on it)
        self._zero_grad = True
        self._pending_tokens = 0
        self.last_grad_norm: Optional[float] = None
        self._grads_fresh: Dict[int, bool] = {}
        attn_layers = [l for l in self.layers if getattr(l, "attn", None) is not None]
        kvh = max((l.attn.cfg.n_kv_heads for l in attn_layers), default=0)
        hd = max((l.attn.cfg.head_dim for l in attn_layers), default=0)
        window = ws.max_seq_len if (attn_layers and ws.max_seq_len > ws.max_chunk_size) else 0
        if window and tp is not None:
            window += 128 * tp.world        # a sequence's last chunk may carry filler tokens up to the shard multiple
        act_dtype = self.layers[0].cfg.dtype if self.layers else torch.bfloat16
        self.buffers = BufferManager(
            [l.param_spec for l in self.layers], embed.param_spec, head.param_spec, optimizer, device,
            n_gpu_layers=ws.n_gpu_layers, n_gpu_grads=ws.n_gpu_grads, n_gpu_opt_layers=ws.n_gpu_opt_layers,
            host_backend=host_backend, kv_window_tokens=window, kv_heads=kvh, head_dim=hd, act_dtype=act_dtype,
            host_act_bytes=ws.host_act_buffer_size, verbose=verbose, **(dp.buffer_kwargs() if dp is not None else {}))
        self.streams = StreamBundle.create(device, secondary=False)
        self.events = EventBook(self.streams)
        # offloaded activations: how many (layer, chunk) slots ahead of the one in backward are being copied back
        import os as _os
        self.act_prefetch_depth = int(_os.environ.get("FTB_ACT_PREFETCH", "2"))
        self._prefetched: Dict = {}
        self._ce = None                 # C++ copy engine, created on first host<->device transfer
        self._ce_key = 0
        self._scheduler = None
        self._last_plan: Optional[SaveLevelPlan] = None
        self.is_causal = True
        self.mrope = any(getattr(l, "attn", None) is not None and l.attn.cfg.rope.mrope_sections for l in self.layers)
        if dp is not None:
            dp.attach(self)
        if ep is not None and hasattr(ep, "attach"):
            ep.attach(self)

    # ====================================================================== public API
    def fwd_bwd(self, seqs: Optional[Seq[Sequence]] = None, loss_scale_factor: Optional[float] = None,
                total_tokens_per_step: Optional[int] = None, loss_fn=None, forward_only: bool = False, *,
                sequences: Optional[Seq[Sequence]] = None, verbose: Optional[bool] = None) -> StepStats:
        """Forward + backward over ``seqs``; gradients accumulate until :meth:`step`.  ``forward_only`` stops after the
        loss (see :meth:`evaluate`): no gradient buffer is read or written.  ``sequences`` is the reference's name for
        the first argument; ``verbose`` overrides the engine's setting for this call."""
        t0 = time.perf_counter()
        if seqs is None:
            seqs = sequences
        if seqs is None:
            raise TypeError("fwd_bwd() needs the step's sequences")
        given = list(seqs)
        seqs = [as_sequence(s) for s in given]                 # any object with ``tokens`` will do
        was_verbose = self.verbose
        if verbose is not None:
            self.verbose = bool(verbose)
        try:
            return self._fwd_bwd(seqs, loss_scale_factor, total_tokens_per_step, loss_fn, forward_only, t0)
        finally:
            self.verbose = was_verbose
            for mine, theirs in zip(seqs, given):              # per-token losses go back to the caller's own objects
                if mine is not theirs and mine.per_token_loss is not None:
                    try:
                        theirs.per_token_loss = mine.per_token_loss
                    except AttributeError:
                        pass

    def _check_sequences(self, seqs) -> None:
        """Host-side checks of what would otherwise be an out-of-range access on the device: a sequence longer than the
        context window the buffers were sized for, a token id outside the embedding table, a target outside the
        vocabulary that is not the ignore value."""
        vocab, limit = int(self.embed.vocab_size), int(self.ws.max_seq_len)
        for s in seqs:
            n = len(s)
            if n == 0:
                raise ValueError(f"sequence {s.seq_id} is empty")
            if n > limit:
                raise ValueError(f"sequence {s.seq_id} has {n} tokens; the model was built with max_seq_len={limit}")
            lo, hi = int(s.tokens.min()), int(s.tokens.max())
            if lo < 0 or hi >= vocab:
                raise ValueError(f"sequence {s.seq_id} has token id {lo if lo < 0 else hi}; the vocabulary has "
                                 f"{vocab} entries")
            t = s.targets
            if t is not None and t.dtype in (torch.int64, torch.int32):
                if len(t) != n:
                    raise ValueError(f"sequence {s.seq_id}: {len(t)} targets for {n} tokens")
                if bool(((t >= vocab) | ((t < 0) & (t != -100))).any()):
                    raise ValueError(f"sequence {s.seq_id} has a target outside [0, {vocab}) that is not -100")
            for name in ("loss_mask", "advantages", "ref_logprobs"):
                extra = getattr(s, name, None)
                if extra is not None and len(extra) != n:
                    raise ValueError(f"sequence {s.seq_id}: {len(extra)} {name} entries for {n} tokens")

    def _fwd_bwd(self, seqs, loss_scale_factor, total_tokens_per_step, loss_fn, forward_only, t0) -> StepStats:
        ws = self.ws
        self._check_sequences(seqs)
        if loss_scale_factor is None:
            loss_scale_factor = 1.0 / max(sum(s.active_token_count for s in seqs), 1)
        total_tokens_per_step = total_tokens_per_step or sum(len(s) for s in seqs)
        rounds = split_sequences(seqs, target_round_tokens=ws.target_round_tokens, max_chunk_size=ws.max_chunk_size,
                                 max_training_chunks=ws.max_training_chunks,
                                 max_total_round_tokens=ws.max_total_round_tokens,
                                 policy=ChunkPolicy.CAUSAL if self.is_causal else ChunkPolicy.NON_CAUSAL)
        if self.ep is not None:
            # expert-parallel ranks exchange rows per (layer, chunk): all of them walk the same number of rounds
            rounds = rounds + [[] for _ in range(self.ep.agree_max(len(rounds)) - len(rounds))]
        stats = StepStats(n_rounds=len(rounds))
        if not forward_only:
            self.fwd_bwd_serial += 1
        loss_acc = torch.zeros((), dtype=torch.float32, device=self.device)
        act_acc = torch.zeros((), dtype=torch.int64, device=self.device)
        pending_losses = []
        with _nvtx("Fwd+Bwd"):
            for r, rseqs in enumerate(rounds):
                with _nvtx(f"Round {r}"):
                    last_round = r == len(rounds) - 1
                    with _nvtx("Prepare Training Chunks"):
                        metas = prepare_training_chunks(rseqs, ws.max_chunk_size, self.device, mrope=self.mrope,
                                                        pad_multiple=128 * self.tp.world if self.tp is not None else 1)
                        if self.ep is not None:
                            metas = self._pad_with_filler_chunks(metas, self.ep.agree_max(len(metas)))
                    with _nvtx("Determine Saved Levels"):
                        plan = self._plan_save_levels(metas)
                    self._last_plan = plan
                    stats.n_chunks += len(metas)
                    stats.tokens += sum(m.num_tokens - m.extra.get("pad_tokens", 0) for m in metas)
                    stats.host_act_bytes = max(stats.host_act_bytes, plan.host_bytes)
                    for k, v in plan.histogram().items():
                        stats.plan_hist[k] = stats.plan_hist.get(k, 0) + v
                    if self._zero_grad and not forward_only:
                        self._zero_all_grads()
                        self._zero_grad = False
                    ctx_base = dict(kv_window=self.buffers.kv_window, total_tokens_per_step=total_tokens_per_step,
                                    tp=self.tp, ep=self.ep,
                                    param_gather=(self.dp.first_gemm if getattr(self.dp, "defer", False) else None))
                    with _nvtx("Setup Round"):
                        if hasattr(self.embed, "setup_round"):           # multimodal: encode the round's images once
                            self.embed.setup_round(rseqs, metas, self.device, train=not forward_only)
                        transitions, slots = self._setup_round(metas)
                    with _nvtx("Forward"):
                        self._forward_pass(metas, plan, transitions, slots, ctx_base, stats)
                    with _nvtx("Head"):
                        for c, meta in enumerate(metas):
                            ls = self.head.forward_backward(transitions[c], self._token_shard(meta),
                                                            self.buffers.head_params(),
                                                            {} if forward_only else self.buffers.head_grads(),
                                                            loss_fn, loss_scale_factor, want_dx=not forward_only)
                            loss_acc += ls.total_loss
                            act_acc += ls.active_tokens
                            pending_losses.append((rseqs, meta, ls.per_token_loss))
                    if forward_only:
                        self.streams.synchronize_all()      # saved activations are dropped: let their copies finish
                    else:
                        with _nvtx("Backward"):
                            self._backward_pass(metas, plan, transitions, slots, ctx_base, stats, last_round)
                        with _nvtx("Embed Backward"):
                            for c, meta in enumerate(metas):
                                self.embed.backward(transitions[c], self._token_shard(meta),
                                                    self.buffers.embed_params(), self.buffers.embed_grads())
                    if hasattr(self.embed, "finalize_round"):
                        self.embed.finalize_round()
                    self.events.clear_per_round()
        if not forward_only:
            self._fold_tied_head_grad()
            if self.dp is not None:
                self.dp.on_embed_head_grads_ready()
        # one host read for the whole call
        stats.loss_sum = float(loss_acc)
        stats.active_tokens = int(act_acc)
        self._write_back_losses(pending_losses)
        if not forward_only:
            self._pending_tokens += stats.tokens
        stats.elapsed_s = time.perf_counter() - t0
        return stats

    # ---- the reference's attribute names (flextrain/engine/active_model.py:175-193)
    @property
    def backbone(self):
        return self.layers

    @property
    def working_set(self) -> WorkingSetConfig:
        return self.ws

    @property
    def hw_cost(self) -> HardwareCost:
        return self.hw

    @property
    def step_count(self) -> int:
        return self.step_num

    @step_count.setter
    def step_count(self, n: int) -> None:
        self.step_num = int(n)

    @property
    def force_saved_act_level(self) -> Optional[int]:
        return self.force_level

    def evaluate(self, seqs: Seq[Sequence], loss_fn=None) -> StepStats:
        """Loss of ``seqs`` under the current weights, forward only: gradients accumulated so far, optimizer state and
        the step counter are untouched (``stats.loss`` is the mean over active tokens; per-token losses are written
        back to the sequences)."""
        return self.fwd_bwd(seqs, loss_scale_factor=1.0, loss_fn=loss_fn, forward_only=True)

    def _fold_tied_head_grad(self) -> None:
        """Tied embeddings are ONE parameter used twice: the head's share of its gradient is added to the embedding's
        before any reduction or update, and the head mirror is refreshed from the embedding after every step
        (:meth:`step`).  Training the mirror separately would untie the model, and an export — which writes the
        embedding only — would lose what the head learnt."""
        if not getattr(self.head, "tied", False):
            return
        ge = self.buffers.embed_grads().get("g_tok_embeddings")
        gh = self.buffers.head_grads().get("g_head_proj")
        if ge is not None and gh is not None:
            ge.add_(gh)
            gh.zero_()

    def grad_norm(self) -> float:
        """Global L2 norm of the accumulated gradients (one host read).  Replicated tensors count once; the parts of
        tensor- / expert-parallel tensors are summed over their group."""
        from .buffers import _views
        bm = self.buffers
        self.streams.synchronize_all()
        dev = self.device
        rep = torch.zeros((), dtype=torch.float32, device=dev)
        part = torch.zeros((), dtype=torch.float32, device=dev)
        units = [(self.embed.param_spec, bm.embed_grads()), (self.head.param_spec, bm.head_grads())]
        for l, layer in enumerate(self.layers):
            g = bm.grads(l) if bm.grads_resident else _views(bm.host_g[l], bm.layers[l].g_layout)
            units.append((layer.param_spec, g))
        if getattr(self.embed, "train_encoders", False):       # a trainable vision tower: replicated, counted once
            for g in self.embed.reduced_encoder_grads(self._encoder_group()).values():
                rep += g.to(torch.float32).pow(2).sum().to(dev)
        for spec, grads in units:
            for t in spec.trainable():
                g = grads.get(t.grad_name)
                if g is None:
                    continue
                sq = g.to(torch.float32).pow(2).sum().to(dev)
                if t.is_local_part:
                    part += sq
                else:
                    rep += sq
        group = self.tp or self.ep
        if group is not None:
            import torch.distributed as dist
            dist.all_reduce(part, group=group.pg)
        return float((rep + part).sqrt())

    def _encoder_group(self):
        """Process group over which a trainable vision tower's gradient is summed: the whole job (data parallel; a
        tower does not combine with tensor parallelism), or ``None`` on one rank."""
        if int(getattr(self, "world_size", 1) or 1) <= 1:
            return None
        import torch.distributed as dist
        return dist.group.WORLD

    def step(self, step_num: Optional[int] = None, *, max_grad_norm: Optional[float] = None) -> int:
        """Optimizer step over embed, head and every layer; returns 0, or the optimizer's error code.
        ``step_num`` is the update's number for AdamW's bias correction (default: one more than the last, as in
        flextrain/engine/active_model.py:428-452); ``max_grad_norm`` scales the gradients down when their global norm
        exceeds it (``last_grad_norm`` keeps the norm before scaling)."""
        self.step_num = self.step_num + 1 if step_num is None else int(step_num)
        grad_scale = 1.0
        sharded = self.dp is not None and getattr(self.dp, "m", None) is not None      # reduced gradients live as shards
        if max_grad_norm is not None:
            self.last_grad_norm = self.dp.grad_norm(self) if sharded else self.grad_norm()
            if self.last_grad_norm > max_grad_norm:
                grad_scale = max_grad_norm / (self.last_grad_norm + 1e-6)
        with _nvtx("Step"):
            if sharded:
                rc = self.dp.step(self, grad_scale)
            elif self.dp is not None:
                rc = self.dp.step(self) if grad_scale == 1.0 else self._step_local(grad_scale)
            else:
                rc = self._step_local(grad_scale)
            if getattr(self.head, "tied", False) and "g_tok_embeddings" in self.buffers.embed_grads():
                self.buffers.head_params()["w_head_proj"].copy_(self.buffers.embed_params()["w_tok_embeddings"])
            if getattr(self.embed, "train_encoders", False):
                rc |= self.embed.step_encoders(self.optimizer, self.step_num, grad_scale, self._encoder_group())
        for l, layer in enumerate(self.layers):
            if self.buffers.params_resident:
                layer.end_of_step(self.buffers.params(l))
        self._zero_grad = True
        self._pending_tokens = 0
        return rc

    # ================================================================= save-level planning
    def _plan_save_levels(self, metas: List[ChunkMeta]) -> SaveLevelPlan:
        nL, nC = len(self.layers), len(metas)
        n_slots = self.ws.n_gpu_act_slots
        if self.force_level is None and nL * nC <= n_slots:
            return SaveLevelPlan.all_on_device(nL, nC)                    # fast path: everything stays in HBM
        toks = [m.num_tokens for m in metas]
        ctxs = [(m.total_k / max(len(m.seq_lens), 1)) / 2 + sum(m.prior_lens) / max(len(m.seq_lens), 1) / 2 for m in metas]
        tables = build_dp_tables(self.layers, toks, self.hw, avg_ctx=ctxs)
        if self.force_level is not None:
            return plan_from_solution(tables, None, nL, nC, n_gpu_act_slots=0 if self.force_level >= 0 else nL * nC,
                                      host_budget_bytes=None, force_level=self.force_level)
        if self._scheduler is None:
            self._scheduler = TransmissionScheduler()
        T = len(tables.tasks)
        pinned = [1 if t >= T - n_slots else 0 for t in range(T)]
        sol, val = self._scheduler.solve(tables.compute_ms, tables.dur_ms, tables.value_ms, n_slots, pinned,
                                         tables.valid_k)
        plan = plan_from_solution(tables, sol, nL, nC, n_gpu_act_slots=n_slots,
                                  host_budget_bytes=self.ws.host_act_buffer_size or None)
        plan.solver_value = val
        if self.verbose:
            print(f"[Save Level Plan] tiers={plan.histogram()} host_bytes={plan.host_bytes / 2**30:.2f} GiB "
                  f"feasible={plan.feasible}")
        return plan

    # ======================================================================= round set-up
    def _setup_round(self, metas):
        self.buffers.reset_host_act()
        transitions = {}
        ep = self.buffers.embed_params()
        for c, meta in enumerate(metas):
            transitions[c] = self.embed.forward(self._token_shard(meta), ep)
        return transitions, {}

    def _pad_with_filler_chunks(self, metas: List[ChunkMeta], n: int) -> List[ChunkMeta]:
        """Append unscored filler chunks until the round has ``n`` chunks (the count of the busiest expert-parallel
        peer).  A filler chunk is a short sequence of its own whose targets are all ``-100``: it joins every
        dispatch / combine of the round, contributes no loss and no gradient (``meta.extra["filler"]`` also keeps it
        out of the router's load-balance term) and is not counted in the step's tokens."""
        if len(metas) >= n:
            return metas
        from ..parallel.ep import FILLER_TOKENS
        next_group = max((m.seq_group for m in metas), default=-1) + 1
        while len(metas) < n:
            toks = torch.zeros(FILLER_TOKENS, dtype=torch.int64)
            fill = Sequence(toks, targets=torch.full((FILLER_TOKENS,), -100, dtype=torch.int64), seq_id=-1)
            m = prepare_training_chunks([fill], self.ws.max_chunk_size, self.device, mrope=self.mrope)[0]
            m.chunk_id = len(metas)
            m.seq_group = next_group
            next_group += 1
            m.extra["pieces"] = []                     # nothing to write back
            m.extra["pad_tokens"] = m.num_tokens       # not part of the step's token count
            m.extra["filler"] = True
            metas.append(m)
        return metas

    def _token_shard(self, meta: ChunkMeta) -> ChunkMeta:
        """Under tensor parallelism the residual stream is token-sharded: the embedding, the head and the loss see
        rows ``[rank * T/tp, (rank+1) * T/tp)`` of the chunk; the layers keep the full chunk's packing metadata."""
        tp = self.tp
        if tp is None:
            return meta
        key = ("_shard", tp.rank)
        cached = meta.extra.get(key)
        if cached is not None:
            return cached
        T, W = meta.num_tokens, tp.world
        if T % (W * 128):
            raise ValueError(f"tensor parallelism needs chunk token counts that are multiples of {W * 128}; got {T} "
                             f"(use sequence lengths / chunk sizes that are multiples of it)")
        a, b = tp.rank * (T // W), (tp.rank + 1) * (T // W)
        cut = lambda t: None if t is None else t[a:b]
        extra = {k: (v[a:b] if k in ("advantages", "ref_logprobs") and v is not None else v)
                 for k, v in meta.extra.items() if not (isinstance(k, tuple) and k[0] == "_shard")}
        sh = dataclasses.replace(meta, tokens=cut(meta.tokens), targets=cut(meta.targets),
                                 loss_mask=cut(meta.loss_mask), extra=extra)
        meta.extra[key] = sh
        return sh

    def _ctx(self, base, meta: Optional[ChunkMeta] = None, **kw) -> LayerContext:
        ctx = LayerContext(**base, **kw)
        if meta is not None and meta.extra.get("filler"):
            ctx.total_tokens_per_step = 0          # a filler chunk takes no part in the load-balance term
        return ctx

    # ============================================================================ forward
    def _forward_pass(self, metas, plan: SaveLevelPlan, transitions, slots, ctx_base, stats: StepStats):
        bm, st, ev = self.buffers, self.streams, self.events
        nL = len(self.layers)
        if not bm.params_resident:
            # events of the previous round are stale; the ring may only be refilled once compute has left it
            ev.weights_in.clear(); ev.layer_out.clear(); ev.grads_in.clear()
            st.wait_stream(st.inbound, st.compute)
            for l in range(min(bm.n_p, nL)):
                self._prefetch_params(l)
        elif not bm.grads_resident:
            ev.layer_out.clear(); ev.grads_in.clear()
        for l, layer in enumerate(self.layers):
            with _nvtx(f"Layer {l}"):
                if not bm.params_resident:
                    ev.weights_in.wait(l, st.compute)
                    st.touch(("p", bm._slot("p", l)), "r", f"forward of layer {l}")
                params = bm.params(l)
                lin_state, lin_conv = {}, {}
                for c, meta in enumerate(metas):
                    slot = ActivationSlot(layer.activation_schema, meta.num_tokens, ON_DEVICE)
                    ctx = self._ctx(ctx_base, meta)
                    if layer.gdn is not None and meta.has_prior:
                        ctx.lin_state_in, ctx.lin_conv_in = lin_state.get(meta.seq_ids[0]), lin_conv.get(meta.seq_ids[0])
                    x = layer.forward(transitions[c], meta, params, slot, ctx)
                    if layer.gdn is not None and any(meta.has_more_chunks):
                        lin_state[meta.seq_ids[0]] = ctx.out.get("lin_state")
                        lin_conv[meta.seq_ids[0]] = ctx.out.get("lin_conv")
                    transitions[c] = x
                    cost = layer.compute_cost(meta.num_tokens, max(meta.total_k / max(len(meta.seq_lens), 1) / 2, 1))
                    stats.fwd_flops += cost.total_fwd_flops
                    stats.attn_fwd_flops += cost.attn_fwd_flops
                    level = plan.level(l, c)
                    if level == ON_DEVICE:
                        slots[(l, c)] = slot
                    else:
                        stats.recompute_flops += (cost.avoided_recompute_flops[-1] - cost.avoided_recompute_flops[
                            min(level, len(cost.avoided_recompute_flops) - 1)])
                        slots[(l, c)] = self._offload_slot(slot, level, l, c)
                if not bm.params_resident:
                    ev.layer_out.record(l, st.compute)
                    nxt = l + bm.n_p
                    if nxt < nL:
                        self._prefetch_params(nxt, after_layer=l)

    # ======================================================================= copy engine
    def _engine_copies(self, pairs, kind: int) -> None:
        """Run ``(dst, src)`` copies through the C++ copy engine, ordered inside the CURRENT stream: the engine's
        worker thread issues one ``cudaMemcpyAsync`` per pair on its own stream after everything queued on the current
        stream so far, and the current stream resumes when the last one has finished.  One Python call per batch
        instead of one ``copy_`` per tensor (flextrain/engine/buffers.py:1088-1164 and
        flextrain/core/activation_schema.py:483-519 issue a ``copy_`` per tensor / field from Python).
        ``FTB_COPY_ENGINE=0`` falls back to ``Tensor.copy_``."""
        if not pairs:
            return
        import os
        if os.environ.get("FTB_COPY_ENGINE", "1") == "0":
            for d, s_ in pairs:
                d.copy_(s_, non_blocking=True)
            return
        if self._ce is None:
            from .copy_engine import CopyEngine
            self._ce = CopyEngine(self.device)
        cur = ev = None
        if self.streams.is_cuda:
            cur = torch.cuda.current_stream(self.device)
            ev = torch.cuda.Event()
            ev.record(cur)
        self._ce_key += 1
        key = self._ce_key
        jobs = [(d, s_, kind, 0, ev, key if i == len(pairs) - 1 else 0) for i, (d, s_) in enumerate(pairs)]
        ticket = self._ce.submit(jobs)
        self._ce.stream_wait(key, ticket, cur)
        self._ce.lib.ftb_ce_forget(self._ce.h, ctypes.c_uint64(key))

    def _ring_copier(self, kind: int):
        return lambda dst, src: self._engine_copies([(dst, src)], kind)

    def _offload_slot(self, slot: ActivationSlot, level: int, l: int, c: int):
        """Send the fields with ``tier <= level`` to the host arena on the outbound stream; drop the rest."""
        bm, st, ev = self.buffers, self.streams, self.events
        if bm.host_act is None:
            slot.demote(level)          # no host arena: keep the saved tiers in HBM, just drop the others
            return slot
        nbytes = slot.schema.home_size_bytes(slot.num_tokens, level)
        hbuf = bm.host_act_slot(nbytes)
        ev.act_computed.record((l, c), st.compute)
        with st.use(st.outbound):
            ev.act_computed.wait((l, c), st.outbound)
            pairs = []
            host = send_home(slot, hbuf, level, copy_fn=lambda d, s_: pairs.append((d, s_)))
            self._engine_copies(pairs, 1)
            st.touch(("hact", hbuf.data_ptr() - bm.host_act.data_ptr()), "w", f"offload of slot ({l}, {c})")
            ev.act_out.record((l, c), st.outbound)
        if st.is_cuda:
            for name in slot.names():
                slot._t[name].record_stream(st.outbound)
        return host

    def _prefetch_params(self, l: int, after_layer: Optional[int] = None):
        bm, st, ev = self.buffers, self.streams, self.events
        with st.use(st.inbound):
            if after_layer is not None:
                ev.layer_out.wait(after_layer, st.inbound)      # ring slot is free once its previous tenant finished
            bm.fetch_layer_params(l, self._ring_copier(0))
            st.touch(("p", bm._slot("p", l)), "w", f"fetch of layer {l}'s parameters (forward)")
            ev.weights_in.record(l, st.inbound)

    # =========================================================================== backward
    def _backward_pass(self, metas, plan, transitions, slots, ctx_base, stats, last_round: bool):
        bm, st, ev = self.buffers, self.streams, self.events
        nL = len(self.layers)
        groups: Dict[int, List[int]] = {}
        for c, m in enumerate(metas):
            groups.setdefault(m.seq_group, []).append(c)
        if not bm.grads_resident:
            # The first layers of this backward pass reuse gradient slots whose last tenants were written back on the
            # outbound stream by the PREVIOUS round (or step): nothing else orders the refill / zeroing of a slot after
            # that copy, so both streams that may write the slot wait for the outbound stream once per pass.
            st.wait_stream(st.compute, st.outbound)
            st.wait_stream(st.inbound, st.outbound)
        # Backward order of the (layer, chunk) slots, for the look-ahead fetch of offloaded activations: while chunk i
        # computes, the host->device copy of the slots of the next ``act_prefetch_depth`` chunks in this order runs on
        # the inbound stream (flextrain/engine/active_model.py:2036-2098 walks backwards the same way and refills the
        # ring slot that was just freed).
        order = [(l, c) for l in range(nL - 1, -1, -1) for g in sorted(groups, reverse=True) for c in reversed(groups[g])]
        pos = {lc: i for i, lc in enumerate(order)}
        depth = self.act_prefetch_depth if bm.host_act is not None else 0
        self._prefetched = {}
        for l in range(nL - 1, -1, -1):
            layer = self.layers[l]
            with _nvtx(f"Layer {l}"):
                if not bm.params_resident:
                    if not ev.weights_in.has(("b", l)) and l + bm.n_p < nL:
                        self._prefetch_params_bwd(l)
                    if ev.weights_in.has(("b", l)):
                        ev.weights_in.wait(("b", l), st.compute)
                    else:
                        ev.weights_in.wait(l, st.compute)
                    st.touch(("p", bm._slot("p", l)), "r", f"backward of layer {l}")
                if not bm.grads_resident:
                    self._prepare_ring_grads(l)
                    st.touch(("g", bm._slot("g", l)), "w", f"backward of layer {l} accumulates gradients")
                params, grads = bm.params(l), bm.grads(l)
                for g in sorted(groups, reverse=True):
                    chunk_ids = groups[g]
                    spans = any(metas[c].has_prior or any(metas[c].has_more_chunks) for c in chunk_ids)
                    if spans and layer.attn is not None:
                        self._refresh_kv_window(l, chunk_ids, metas, slots)
                    lin_d = {}
                    for c in reversed(chunk_ids):
                        meta = metas[c]
                        i = pos[(l, c)]
                        for nl, nc in order[i + 1: i + 1 + depth]:       # start the copies of the chunks that follow
                            self._issue_fetch(slots, nl, nc)
                        slot = self._fetch_slot(slots.pop((l, c)), l, c)
                        ctx = self._ctx(ctx_base, meta)
                        if layer.gdn is not None:
                            if meta.has_prior:
                                prev = self._peek_slot(slots[(l, c - 1)])
                                ctx.lin_state_in = prev._t["lin_final_state"].to(self.device)
                                ctx.lin_conv_in = prev._t["lin_conv_state"].to(self.device)
                            if any(meta.has_more_chunks):
                                ctx.lin_dstate_in, ctx.lin_dconv_in = lin_d.get("s"), lin_d.get("c")
                        with _nvtx(f"Recompute: Chunk {c}"):
                            layer.forward_recompute(meta, params, slot, ctx)
                        with _nvtx(f"Backward: Chunk {c}"):
                            transitions[c] = layer.backward(transitions[c], meta, params, grads, slot, ctx)
                        if layer.gdn is not None:
                            lin_d = {"s": ctx.out.get("lin_dstate"), "c": ctx.out.get("lin_dconv")}
                        del slot
                ev.grads_ready.record(l, st.compute)
                if not bm.grads_resident:
                    with st.use(st.outbound):
                        ev.grads_ready.wait(l, st.outbound)
                        bm.offload_layer_grads(l, self._ring_copier(1))
                        st.touch(("g", bm._slot("g", l)), "r", f"write-back of layer {l}'s gradients")
                        ev.layer_out.record(("g", l), st.outbound)
                if not bm.params_resident:
                    ev.layer_out.record(("b", l), st.compute)
                    nxt = l - bm.n_p
                    if nxt >= 0:
                        self._prefetch_params_bwd(nxt, after=("b", l))
                if self.dp is not None and last_round:
                    self.dp.on_layer_grads_ready(l)
        self._prefetched = {}

    def _prefetch_params_bwd(self, l: int, after=None):
        bm, st, ev = self.buffers, self.streams, self.events
        with st.use(st.inbound):
            if after is not None:
                ev.layer_out.wait(after, st.inbound)
            bm.fetch_layer_params(l, self._ring_copier(0))
            st.touch(("p", bm._slot("p", l)), "w", f"fetch of layer {l}'s parameters (backward)")
            ev.weights_in.record(("b", l), st.inbound)

    def _prepare_ring_grads(self, l: int):
        """Ring-resident gradients: zero the slot on the first round of a step, else bring the partial sums back."""
        bm, st, ev = self.buffers, self.streams, self.events
        prev_tenant = l + bm.n_g
        if ev.layer_out.has(("g", prev_tenant)):
            ev.layer_out.wait(("g", prev_tenant), st.compute)
        if self._grads_fresh.get(l, True):
            bm.zero_layer_grads(l)
            st.touch(("g", bm._slot("g", l)), "w", f"zero of layer {l}'s gradient slot")
            self._grads_fresh[l] = False
        else:
            with st.use(st.inbound):
                if ev.layer_out.has(("g", prev_tenant)):
                    ev.layer_out.wait(("g", prev_tenant), st.inbound)
                bm.fetch_layer_grads(l, self._ring_copier(0))
                st.touch(("g", bm._slot("g", l)), "w", f"fetch of layer {l}'s partial gradients")
                ev.grads_in.record(l, st.inbound)
            ev.grads_in.wait(l, st.compute)

    def _peek_slot(self, slot):
        return slot

    def _issue_fetch(self, slots, l: int, c: int) -> None:
        """Start the host->device copy of an offloaded slot on the inbound stream without making compute wait for it
        (look-ahead).  The device copy is parked in ``_prefetched`` until :meth:`_fetch_slot` picks it up; the host slot
        stays in ``slots`` (the K/V window refresh and the recurrent-state hand-over of Gated DeltaNet read from it)."""
        slot = slots.get((l, c))
        if slot is None or (l, c) in self._prefetched or slot.buffer is None or slot.buffer.device == self.device:
            return
        st, ev = self.streams, self.events
        with st.use(st.inbound):
            ev.act_out.wait((l, c), st.inbound)
            pairs = []
            dev = fetch_home(slot, None, self.device, copy_fn=lambda d, s_: pairs.append((d, s_)))
            self._engine_copies(pairs, 0)
            if self.buffers.host_act is not None:
                st.touch(("hact", slot.buffer.data_ptr() - self.buffers.host_act.data_ptr()), "r",
                         f"fetch of slot ({l}, {c})")
            ev.act_in.record((l, c), st.inbound)
        self._prefetched[(l, c)] = dev

    def _fetch_slot(self, slot: ActivationSlot, l: int, c: int) -> ActivationSlot:
        """Bring an offloaded slot back into HBM at its saved level (stale higher tiers stay invisible).  If the copy
        was started ahead of time by :meth:`_issue_fetch` only its completion is awaited."""
        st, ev = self.streams, self.events
        if slot.buffer is None or slot.buffer.device == self.device:
            return slot
        dev = self._prefetched.pop((l, c), None)
        if dev is None:
            self._issue_fetch({(l, c): slot}, l, c)
            dev = self._prefetched.pop((l, c))
        ev.act_in.wait((l, c), st.compute)
        if st.is_cuda:
            # allocated while the inbound stream was current, consumed on the compute stream: the allocator must not
            # hand this memory to the next inbound allocation before compute is done with it
            for name in dev.names():
                dev._t[name].record_stream(st.compute)
        return dev

    def _refresh_kv_window(self, l: int, chunk_ids, metas, slots) -> None:
        """Refill the rolling K/V window with layer ``l``'s saved K/V of every chunk of a multi-chunk sequence and
        clear the dK/dV accumulators (flextrain/engine/active_model.py:1941-2034)."""
        w = self.buffers.kv_window
        st = self.streams
        live = 0
        with st.use(st.inbound_fwd_context):
            st.wait_stream(st.inbound_fwd_context, st.compute)
            st.touch(("kv",), "w", f"K/V window refill for layer {l}")
            for c in chunk_ids:
                m = metas[c]
                if not (m.has_prior or any(m.has_more_chunks)):
                    continue
                P, L = m.prior_lens[0], m.seq_lens[0]
                s = self._prefetched.get((l, c))
                if s is not None:                         # already on its way back to HBM: take K/V from that copy
                    self.events.act_in.wait((l, c), st.inbound_fwd_context)
                else:
                    s = slots[(l, c)]
                    if self.events.act_out.has((l, c)):   # saved K/V live in the host arena: wait for their arrival
                        self.events.act_out.wait((l, c), st.inbound_fwd_context)
                w.k[P:P + L].copy_(s._t["xk"], non_blocking=True)
                w.v[P:P + L].copy_(s._t["xv"], non_blocking=True)
                live = max(live, P + L)
            # only the keys this group can see collect dK / dV: clear that range, not the whole window
            w.dk[:live].zero_()
            w.dv[:live].zero_()
        st.wait_stream(st.compute, st.inbound_fwd_context)
        st.touch(("kv",), "w", f"backward of layer {l} over the K/V window")

    # =============================================================================== step
    def _step_local(self, grad_scale: float = 1.0) -> int:
        bm, st, ev = self.buffers, self.streams, self.events
        opt, rc = self.optimizer, 0
        rc |= opt.step(self.embed.param_spec, bm.embed_params(), bm.embed_grads(), bm.embed_opt(), self.step_num,
                       grad_scale)
        rc |= opt.step(self.head.param_spec, bm.head_params(), bm.head_grads(), bm.head_opt(), self.step_num,
                       grad_scale)
        if rc:
            return rc
        nL = len(self.layers)
        ringed = not (bm.params_resident and bm.grads_resident and bm.opt_resident)
        if not ringed:
            for l, layer in enumerate(self.layers):
                rc |= opt.step(layer.param_spec, bm.params(l), bm.grads(l), bm.opt_state(l), self.step_num, grad_scale)
                if rc:
                    return rc
            return rc
        # ---- streamed step: prefetch k+depth on inbound, update on compute, write back on outbound
        ring_n = [n for n, res in ((bm.n_p, bm.params_resident), (bm.n_g, bm.grads_resident),
                                   (max(bm.n_o, 2), bm.opt_resident)) if not res]
        depth = min(ring_n + [nL])

        def fetch(k):
            # a ring slot may be refilled once its previous tenant (k - n) has been written back
            with st.use(st.inbound):
                for n in ring_n:
                    if k - n >= 0:
                        ev.layer_out.wait(("s", k - n), st.inbound)
                cp = self._ring_copier(0)
                bm.fetch_layer_params(k, cp); bm.fetch_layer_grads(k, cp); bm.fetch_layer_opt(k, cp)
                for kind, res in (("p", bm.params_resident), ("g", bm.grads_resident), ("o", bm.opt_resident)):
                    if not res:
                        st.touch((kind, bm._slot(kind, k)), "w", f"fetch of layer {k}'s {kind} state for the update")
                ev.opt_in.record(k, st.inbound)

        st.wait_stream(st.inbound, st.compute)
        st.wait_stream(st.inbound, st.outbound)
        for k in range(min(depth, nL)):
            fetch(k)
        for l, layer in enumerate(self.layers):
            ev.opt_in.wait(l, st.compute)
            for kind, res, mode in (("p", bm.params_resident, "w"), ("g", bm.grads_resident, "r"),
                                    ("o", bm.opt_resident, "w")):
                if not res:
                    st.touch((kind, bm._slot(kind, l)), mode, f"optimizer update of layer {l}")
            rc |= opt.step(layer.param_spec, bm.params(l), bm.grads(l), bm.opt_state(l), self.step_num, grad_scale)
            if rc:
                break
            layer.end_of_step(bm.params(l))
            ev.layer_out.record(("c", l), st.compute)
            with st.use(st.outbound):
                ev.layer_out.wait(("c", l), st.outbound)
                bm.offload_layer_params(l, self._ring_copier(1))
                bm.offload_layer_opt(l, self._ring_copier(1))
                for kind, res in (("p", bm.params_resident), ("o", bm.opt_resident)):
                    if not res:
                        st.touch((kind, bm._slot(kind, l)), "r", f"write-back of layer {l}'s {kind} state")
                ev.layer_out.record(("s", l), st.outbound)
            if l + depth < nL:
                fetch(l + depth)
        st.synchronize_all()
        ev.weights_in.clear(); ev.layer_out.clear(); ev.opt_in.clear()
        self._grads_fresh = {}
        return rc

    # ============================================================================= helpers
    def _zero_all_grads(self) -> None:
        bm = self.buffers
        bm.embed_g.zero_()
        bm.head_g.zero_()
        if getattr(self.embed, "train_encoders", False):
            self.embed.zero_encoder_grads()
        if bm.grads_resident:
            for b in bm.gpu_g:
                b.zero_()
        self._grads_fresh = {}

    def _write_back_losses(self, pending) -> None:
        """Per-token losses back into each ``Sequence`` (flextrain/engine/active_model.py:1306-1312)."""
        for rseqs, meta, per_tok in pending:
            if self.tp is not None:
                per_tok = self.tp.all_gather(per_tok)          # each rank computed the losses of its token shard
            host = per_tok.detach().to("cpu")
            off = 0
            for i, start, n in meta.extra["pieces"]:
                s = rseqs[i]
                if s.per_token_loss is None:
                    s.per_token_loss = torch.zeros(len(s), dtype=torch.float32)
                s.per_token_loss[start:start + n] = host[off:off + n]
                off += n

    def synchronize(self) -> None:
        self.streams.synchronize_all()

    def protocol_violations(self) -> List[str]:
        """Ordering violations found by the host-side stream-protocol checker (``FTB_STREAM_CHECK=1``): every ring
        slot, host-arena range or K/V-window access that is not ordered after the accesses it conflicts with."""
        chk = self.streams.checker
        return [] if chk is None else [str(v) for v in chk.violations]

    def check_health(self, error_words=None) -> None:
        """Raise if anything on the device gave up during the step that just ran.

        The kernels never spin for ever: a wait on a peer's flag, an mbarrier or an arrival counter stops after its
        limit, records an error word and lets the kernel return, so the step "finishes" with incomplete data (a
        reduce-scatter that summed gradients a peer had not finished writing, an optimizer that then pushed the
        result to every rank).  The host therefore reads the words after every step and stops the run.  Call it after
        :meth:`step`; it synchronises this rank's streams.  ``error_words`` replaces the read of the kernel libraries
        (host-side tests inject a fake status through it)."""
        self.streams.synchronize_all()
        if error_words is None:
            if self.device.type == "cuda":
                from ..ops.cuda import device_error_words
                error_words = device_error_words()
            else:
                error_words = {}
        bad = {k: v for k, v in error_words.items() if v}
        if bad:
            raise RuntimeError(f"device-side wait or check failed during step {self.step_num}: {bad} "
                               "(library: code*1000 + site); gradients / parameters of this step are not trustworthy")
        for grp in (self.dp, self.ep, self.tp):
            if grp is not None and hasattr(grp, "check"):
                grp.check()

    # --------------------------------------------------------------------- HF load / save
    def load_hf(self, model_dir: Optional[str] = None, strict: bool = False, *, hf_path: Optional[str] = None,
                arch=None) -> None:
        """Fill the master weights from an HF directory.  ``hf_path`` is the reference's name for the directory; the
        family's name map is found from the model's own configuration, so ``arch`` is accepted and not needed."""
        from ..io.hf_weights import load_hf_into_model
        load_hf_into_model(self, model_dir or hf_path, strict=strict)

    def save_hf(self, out_dir: str, filename: Optional[str] = None, *, out_filename: Optional[str] = None,
                arch=None) -> str:
        """One safetensors file of the weights the engine holds, in checkpoint names; returns its path
        (flextrain/engine/active_model.py:795-840; ``out_filename`` is the reference's name for ``filename``)."""
        from ..io.hf_weights import export_model_safetensors
        return export_model_safetensors(self, out_dir, filename or out_filename or "final.safetensors")

    def save_training_state(self, out_dir: str, extra: Optional[dict] = None) -> str:
        """Weights + optimizer state + step counter (every rank calls it); see ``io/training_state.py``."""
        from ..io.training_state import save_training_state
        return save_training_state(self, out_dir, extra)

    def load_training_state(self, src_dir: str, strict: bool = True) -> dict:
        from ..io.training_state import load_training_state
        return load_training_state(self, src_dir, strict)

    def named_master_params(self):
        """Yield ``(scope, layer_index, name, tensor)`` over every master tensor (embed, layers, head)."""
        for n, t in self.buffers.embed_params().items():
            yield "embed", -1, n, t
        for l in range(len(self.layers)):
            for n, t in self.buffers.host_params(l).items():
                yield "layer", l, n, t
        for n, t in self.buffers.head_params().items():
            yield "head", -1, n, t

    def spec_of(self, scope: str, layer: int, name: str):
        """The :class:`TensorSpec` behind one item of :meth:`named_master_params`."""
        ps = {"embed": self.embed, "head": self.head}.get(scope) or self.layers[layer]
        return ps.param_spec.get(name)

    def push_masters_to_device(self) -> None:
        """After editing host masters of a ringed model (load / init), nothing else is needed: layers are fetched
        from the masters on demand.  Resident models are edited in place."""
        return None

    def destroy(self) -> None:
        if self._ce is not None:
            self._ce.synchronize()
            self._ce.close()
            self._ce = None
        self.buffers.destroy()
