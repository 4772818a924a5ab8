"""Headline benchmark: trained tokens/s for the whole job, Llama-3.1-8B full fine-tune.

    python bench.py --gpus 1 --steps 2 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...          # the unmodified reference engine, same metric and config

Config (fixed): 32 layers, hidden 4096, 32 query / 8 KV heads, head_dim 128, SwiGLU 14336, vocab 128256, RoPE
theta 5e5; bf16 weights / activations / gradients, fp32 AdamW state; synthetic uniform tokens, seq_len 1024,
global batch 524288 tokens per optimizer step (strong scaling: the global batch is split over the GPUs);
random-init weights.  Every timed step runs forward, backward, the data-parallel gradient reduction and the
optimizer update.  ONE timed region of K steps after W warm-up steps; each iteration draws its tokens on the host,
puts them in pinned memory, and goes through the public API (``fwd_bwd`` copies them to the device, ``step``
updates, the loss is read back).  CUDA events around the loop give ``value`` (max over ranks), the wall clock
around the same loop gives ``e2e``.  Every GPU count trains on the same global batch (one seeded host stream,
rank r keeps sequences r, r + N, ...), so ``loss_step1`` is comparable across N.  If K steps do not fit the wall
budget of the process (``--budget-s``), fewer are timed and ``steps`` reports the count that ran.
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA31_8B = dict(vocab_size=128256, n_layers=32, d_model=4096, n_heads=32, n_kv_heads=8, head_dim=128,
                  expert_dim=14336, ffn_dim=14336, num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)
SEQ_LEN = 1024
GLOBAL_BATCH = 524288
# The other named configurations (``--config``); the headline stays llama8b.
CONFIGS = {
    "llama8b": dict(model="Llama-3.1-8B", arch="llama", dims=LLAMA31_8B, seq_len=SEQ_LEN, global_batch=GLOBAL_BATCH,
                    hyper={"rope_theta": 500000.0, "norm_eps": 1e-5}, scaling="strong", published=3733.0),
    # LoRA r16 on every linear of the same model (reference: 5,295 tokens/s on an RTX 5090, docs/verified_runs.md:159)
    "llama8b_lora": dict(model="Llama-3.1-8B", arch="llama", dims=LLAMA31_8B, seq_len=SEQ_LEN, global_batch=GLOBAL_BATCH,
                         hyper={"rope_theta": 500000.0, "norm_eps": 1e-5}, scaling="strong", published=5295.0,
                         lora=dict(targets="all", rank=16, alpha=16.0)),
    # long-context dense 12B: one 32768-token sequence per GPU (weak scaling), chunked attention with a KV window
    "longctx12b": dict(model="dense-12B long context", arch="llama",
                       dims=dict(vocab_size=131072, n_layers=40, d_model=5120, n_heads=32, n_kv_heads=8, head_dim=128,
                                 expert_dim=14336, ffn_dim=14336, num_routed_experts=0, num_shared_experts=0, top_k=0,
                                 is_causal=True),
                       seq_len=32768, per_gpu_batch=32768, hyper={"rope_theta": 1000000.0, "norm_eps": 1e-5},
                       scaling="weak"),
    # OLMoE-1B-7B on one GPU: 64 experts, top-8 (reference: 13,346 tokens/s full FT on an RTX 5090,
    # docs/verified_runs.md:161); the single-GPU MoE path (device-side routing plan, grouped tcgen05 GEMMs)
    "olmoe1b7b": dict(model="OLMoE-1B-7B", arch="olmoe",
                      dims=dict(vocab_size=50304, n_layers=16, d_model=2048, n_heads=16, n_kv_heads=16, head_dim=128,
                                expert_dim=1024, ffn_dim=1024, num_routed_experts=64, num_shared_experts=0, top_k=8,
                                is_causal=True),
                      seq_len=2048, global_batch=262144, hyper={"rope_theta": 10000.0, "norm_eps": 1e-5},
                      scaling="strong", published=13346.0),
    # Qwen3-MoE 30B-A3B: experts sharded over all GPUs (expert parallel), the rest data parallel
    "qwen3moe30b": dict(model="Qwen3-30B-A3B", arch="qwen3_moe",
                        dims=dict(vocab_size=151936, n_layers=48, d_model=2048, n_heads=32, n_kv_heads=4, head_dim=128,
                                  expert_dim=768, ffn_dim=768, num_routed_experts=128, num_shared_experts=0, top_k=8,
                                  is_causal=True),
                        seq_len=4096, global_batch=262144, hyper={"rope_theta": 1000000.0, "norm_eps": 1e-6},
                        scaling="strong", ep="world"),
    # Llama-3-70B architecture: tensor parallel over all GPUs
    "llama70b": dict(model="Llama-3-70B", arch="llama",
                     dims=dict(vocab_size=128256, n_layers=80, d_model=8192, n_heads=64, n_kv_heads=8, head_dim=128,
                               expert_dim=28672, ffn_dim=28672, num_routed_experts=0, num_shared_experts=0, top_k=0,
                               is_causal=True),
                     seq_len=2048, global_batch=262144, hyper={"rope_theta": 500000.0, "norm_eps": 1e-5},
                     scaling="strong", tp="world", opt_state="host"),
}
PUBLISHED_TOK_S = 3733.0          # reference, RTX 5090, Llama-3.1-8B full FT (docs/verified_runs.md:160)
METRIC = "train tokens/sec/box, Llama-3.1-8B full FT"


class ClockSampler:
    """Samples SM clocks and throttle reasons of this rank's GPU with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "200", "-i", str(gpu_index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except Exception:
            self.p = None

    def stop(self) -> dict:
        if self.p is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except Exception:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        for line in self.f.read().splitlines():
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1])); mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        try:
            os.unlink(self.f.name)
        except OSError:
            pass
        # the busiest half of the samples is "under load"
        load = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def _dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


_JSON_FD = None


def _claim_stdout() -> None:
    """Keep file descriptor 1 for the one JSON line: a duplicate of it is kept for ``_emit`` and descriptor 1 itself is
    pointed at stderr, so whatever else writes to stdout in this process (library banners such as NCCL's version line,
    the reference's planner notes, C extensions) lands in the log instead of in front of the result."""
    global _JSON_FD
    if _JSON_FD is None:
        sys.stdout.flush()
        _JSON_FD = os.dup(1)
        os.dup2(2, 1)


def _emit(obj):
    line = (json.dumps(obj) + "\n").encode()
    if _JSON_FD is None:
        sys.__stdout__.write(line.decode())
        sys.__stdout__.flush()
    else:
        os.write(_JSON_FD, line)


def _budget_steps(args, t_proc0: float, warm_step_s: float, setup_reserve_s: float = 25.0) -> int:
    """Number of timed steps that fit into the wall-clock budget of this process (``--budget-s``, default 800 s:
    the scaling run gives every command 870 s).  The requested count is used whenever it fits."""
    if args.budget_s <= 0 or warm_step_s <= 0:
        return args.steps
    left = args.budget_s - (time.perf_counter() - t_proc0) - setup_reserve_s
    fit = int(left // warm_step_s)
    return max(min(args.steps, fit), min(args.steps, 3))


def run_ours(args):
    t_proc0 = time.perf_counter()
    os.environ.setdefault("FTB_STRICT", "1")        # a library fallback on a hot op raises instead of running
    import torch
    import torch.distributed as dist

    import flextrain_b200 as ft
    from flextrain_b200 import ops
    from flextrain_b200.io.sequence import Sequence
    from flextrain_b200.ops import cuda as kernels

    rank, world, local = _dist_env()
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(dev))
    cfg = CONFIGS[args.config]
    dims = dict(cfg["dims"])
    seq_len = cfg["seq_len"]
    gbatch = cfg.get("global_batch") or cfg["per_gpu_batch"] * world
    if args.small:                          # debugging only; never used for a reported number
        dims.update(n_layers=4)
        gbatch = 65536 if "global_batch" in cfg else gbatch
    par = {k: (world if cfg.get(k) == "world" else 1) for k in ("tp", "ep")}
    # tensor parallel ranks work on the same tokens (each feeds the whole batch); data parallel ranks split it
    dp = 1 if par["tp"] > 1 else world
    per_rank = gbatch // dp
    free, total = torch.cuda.mem_get_info()
    lora = cfg.get("lora")
    opt = ft.AdamW(lr=1e-4 if lora else 3e-5, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0,
                   state_dtype=torch.float32)
    extra = dict(lora_targets=lora["targets"], lora_rank=lora["rank"], lora_alpha=lora["alpha"]) if lora else {}
    host_bytes = args.host_gib << 30
    if cfg.get("opt_state") == "host" and not args.opt_state_device:
        # fp32 AdamW state of the rank's slice lives in pinned host memory: give the planner this rank's share of it
        import psutil
        host_bytes = max(host_bytes, int(psutil.virtual_memory().available * 0.8) // max(world, 1))
        extra["opt_state"] = "host"
    am = ft.from_dims(dims, arch=cfg["arch"], optimizer=opt, max_seq_len=seq_len, max_global_batch_tokens=gbatch,
                      max_gpu_mem_bytes=int(free), max_host_mem_bytes=host_bytes, device=dev,
                      hyperparams=cfg["hyper"], world_size=world, rank=rank,
                      dp_shard=args.shard, init_on_device=True, init_std=0.02, verbose=(rank == 0 and args.verbose),
                      max_chunk_size=args.chunk, head_chunk_size=args.head_chunk, **par, **extra)
    # one seeded host stream for the whole job, so the global batch (and the loss) is the same at every GPU count
    src = ft.SyntheticTokenSource(dims["vocab_size"], seq_len, seed=1234, pin=False)
    n_global = gbatch // seq_len
    h2d = [0]

    def next_batch():
        """Host side of a step: draw the global batch, keep this rank's sequences, put them in pinned memory."""
        seqs = src.get_sequences(gbatch)
        assert len(seqs) == n_global
        mine = seqs[rank % dp::dp]
        out = [Sequence(s.tokens.pin_memory(), targets=s.targets.pin_memory(), seq_id=s.seq_id) for s in mine]
        h2d[0] = sum(s.tokens.numel() * 8 + s.targets.numel() * 8 for s in out)
        return out

    def one_step(seqs):
        st = am.fwd_bwd(seqs, loss_scale_factor=1.0 / gbatch, total_tokens_per_step=gbatch)   # H2D of tokens/targets
        rc = am.step()
        assert rc == 0
        return st                                    # st.loss was read back from the device (D2H)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    loss_step1, warm_s = None, 0.0
    for i in range(args.warmup):
        barrier()
        t0 = time.perf_counter()
        st = one_step(next_batch())
        barrier()
        warm_s = time.perf_counter() - t0           # the last warm-up step is the estimate for the budget
        if i == 0:
            loss_step1 = st.loss
    peak_alloc = torch.cuda.max_memory_allocated() / 2 ** 30
    steps = _budget_steps(args, t_proc0, warm_s)
    if world > 1:
        tsteps = torch.tensor([steps], device=dev)
        dist.all_reduce(tsteps, op=dist.ReduceOp.MIN)
        steps = int(tsteps.item())

    # ---- ONE timed region: CUDA events give ``value``, the wall clock around the same loop gives ``e2e``.
    # Every iteration draws its tokens on the host, copies them from pinned memory, trains, reads the loss back.
    sampler = ClockSampler(local)
    ops.reset_launch_count()
    ops.reset_backends_used()
    if args.op_timing:
        ops.enable_op_timing()
        ops.reset_op_timing()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in range(steps):
        st = one_step(next_batch())
    e1.record()
    barrier()
    e2e_s = time.perf_counter() - t0
    dev_ms = e0.elapsed_time(e1)
    launches = ops.launch_count()
    clocks = sampler.stop()
    last_loss = st.loss

    t = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(t[0]), float(t[1])
    if args.op_timing and rank == 0:
        rows = ops.timing_report()
        with open(args.op_timing, "w") as f:
            json.dump({"steps": steps, "device_ms": dev_ms, "ops_ms": sum(r["total_ms"] for r in rows), "rows": rows}, f,
                      indent=1)
    errs = kernels.device_error_words()
    am.check_health()                                # raises when a bounded device-side wait ran out
    if rank == 0:
        ms_step = dev_ms / steps
        value = gbatch / (ms_step / 1e3)
        e2e_val = gbatch / (e2e_ms / steps / 1e3)
        n_params = 0
        for scope, l, name, t in am.named_master_params():
            sp = am.spec_of(scope, l, name)
            if sp.shard.ep_dim is not None:       # routed experts: only top_k of num_experts are active per token
                n_params += t.numel() * par["ep"] * dims["top_k"] // dims["num_routed_experts"]
            else:
                n_params += t.numel() * (par["tp"] if sp.is_local_part else 1)
        flops_tok = 6.0 * (n_params - dims["vocab_size"] * dims["d_model"]) \
            + 6.0 * seq_len * dims["n_heads"] * dims["head_dim"] * dims["n_layers"]
        if lora:                                  # frozen base: no weight-gradient GEMMs (4 of the 6 FLOPs per weight)
            flops_tok = flops_tok * 4.0 / 6.0
        tflops_gpu = value * flops_tok / world / 1e12
        peaks = {}
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
        except Exception:
            pass
        sustained = peaks.get("bf16_tflops_sustained", 1400.0)
        headline = args.config == "llama8b"
        _emit({
            "metric": METRIC if headline else f"train tokens/sec/box, {cfg['model']} {'LoRA' if lora else 'full FT'}",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": cfg["scaling"],
            "vs_baseline": value / cfg["published"] if cfg.get("published") else None, "dtype": "bf16",
            "data": "synthetic uniform tokens, random-init weights",
            "config": {"model": cfg["model"] + (" (SMALL DEBUG)" if args.small else ""), "global_batch": gbatch,
                       "seq_len": seq_len, "parallelism": (f"tp{world}" if par["tp"] > 1 else f"dp{world}" + (f"+ep{world}" if par["ep"] > 1 else ""))
                       + (f"-shard({am.ws.shard})" if world > 1 else ""),
                       "optimizer": "AdamW fp32 state",
                       "opt_state": "host" if am.ws.n_gpu_opt_layers is not None else "hbm",
                       "round_tokens": am.ws.target_round_tokens,
                       "chunk": am.ws.max_chunk_size, "rounds_per_step": am.ws.target_num_rounds,
                       "l2": "inputs larger than L2 (each step streams >100 GB of weights/activations)",
                       "backends": ops.backends_used(), "strict": os.environ.get("FTB_STRICT") == "1",
                       "timed_region": "one loop: host token draw -> pinned -> H2D -> fwd_bwd -> step -> D2H loss; "
                                       "CUDA events and wall clock bracket the same steps"},
            "steps_requested": args.steps, "diagnostic_op_timing": bool(args.op_timing),
            "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": h2d[0],
                    "d2h_bytes_per_step": 4 * per_rank + 12},
            "gpu_launches": launches,
            "model_tflops_per_gpu": tflops_gpu, "pct_of_measured_sustained_bf16": 100.0 * tflops_gpu / sustained,
            "loss": last_loss, "loss_step1": loss_step1, "peak_alloc_gib": peak_alloc, "device_errors": errs,
        })
    if world > 1:
        dist.destroy_process_group()


def _host_memory_report() -> dict:
    """What the box offers (psutil and the cgroup limit), printed to stderr by the reference arm for diagnosis."""
    out = {}
    try:
        import psutil
        vm = psutil.virtual_memory()
        out.update(total_gib=vm.total / 2 ** 30, available_gib=vm.available / 2 ** 30)
    except Exception:
        pass
    for p in ("/sys/fs/cgroup/memory.max", "/sys/fs/cgroup/memory/memory.limit_in_bytes"):
        try:
            v = open(p).read().strip()
            out["cgroup_limit_gib"] = None if v == "max" else int(v) / 2 ** 30
            break
        except Exception:
            continue
    return out


def _device_of(local: int) -> str:
    """Device string of this rank (one place, so a test can walk the reference arm's control flow on CPU ranks)."""
    return f"cuda:{local}"


def run_reference(args):
    """The unmodified reference engine (installed under baseline/_ref) through its own public API
    (``flextrain.from_dims`` -> ``fwd_bwd`` -> ``step``): same model, sequence length, batch and optimizer."""
    t_proc0 = time.perf_counter()
    rank, world, local = _dist_env()
    ref_root = os.path.join(ROOT, "baseline", "_ref")

    def unavailable(why: str):
        if rank == 0:
            _emit({"impl": "reference", "unavailable": why[:300].replace("\n", " ")})
        sys.exit(0)

    if not os.path.isdir(os.path.join(ref_root, "flextrain")):
        unavailable("baseline/_ref/flextrain is missing: the reference was not installed on this box")
    sys.path.insert(0, ref_root)
    try:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dev = _device_of(local)
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device(dev))
        import flextrain as ref
        from flextrain.core import _memory as ref_memory
        from flextrain.core.hw_probe import probe_hardware
        from flextrain.core.save_level import HardwareCost
        from flextrain.io.sequence import Sequence as RefSequence
        from flextrain.io.sources import SyntheticTokenSource
        from flextrain.optim.adamw import AdamW, AdamWHyperparams
    except Exception as e:
        unavailable(f"reference import failed: {type(e).__name__}: {e}")
    try:
        # only the keys the reference's Llama adapter documents; its own defaults fill the rest (a dense FFN is
        # "one shared expert" there: num_shared_experts = 1, flextrain/io/arch/llama.py:154-159)
        dims = {k: LLAMA31_8B[k] for k in ("vocab_size", "n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim",
                                           "expert_dim")}
        seq_len, gbatch = SEQ_LEN, GLOBAL_BATCH
        if args.small:
            dims["n_layers"] = 4
            gbatch = 65536
        per_rank = gbatch // world
        free, _ = torch.cuda.mem_get_info()
        # The reference pins its whole host budget (cudaHostRegister), so the budget must be something the box can
        # pin: its own cgroup-aware figure, split over the ranks of the node, capped at the 192 GiB host of its
        # published runs (docs/verified_runs.md:141-155).
        host_avail = int(ref_memory.get_available_host_memory())
        host_budget = min(int(host_avail * 0.85) // max(world, 1), 192 << 30)
        if rank == 0:
            print(f"[reference arm] host memory: {_host_memory_report()} reference sees "
                  f"{host_avail / 2 ** 30:.1f} GiB -> budget {host_budget / 2 ** 30:.1f} GiB per rank; "
                  f"GPU free {free / 2 ** 30:.1f} GiB", file=sys.stderr, flush=True)
        probe = probe_hardware(device=dev)          # once (about 10 s); every planning attempt reuses it
        hw_probed = (probe.hw_cost, probe.mem_bw_gbps)
        # second choice when the probed figures make the planner's round target unplannable (a slow shared PCIe
        # link inflates it): nominal B200 host link and the probed compute
        hw_nominal = (HardwareCost(peak_tflops=probe.hw_cost.peak_tflops, pcie_bw_gbps=50.0), probe.mem_bw_gbps)
        if rank == 0:
            print(f"[reference arm] probe: {probe.hw_cost.peak_tflops:.0f} TFLOP/s, PCIe "
                  f"{probe.hw_cost.pcie_bw_gbps:.1f} GB/s, memory {probe.mem_bw_gbps:.0f} GB/s",
                  file=sys.stderr, flush=True)
        # Plan ladder through public keywords only.  The reference's search is tuned for 24-32 GiB cards
        # (flextrain/core/working_set.py:1684-1736): when it rejects its own candidates on a 180 GB GPU, offer a
        # smaller chunk cap, then a smaller GPU budget, then the nominal link figure, then its default bf16
        # optimizer state; the first plan that builds is the one that runs, and the JSON line says which.
        src = SyntheticTokenSource(dims["vocab_size"], seq_len, seed=1234)

        def next_batch():
            seqs = src.get_sequences(gbatch)
            return seqs[rank::world]

        def allreduce_grads():
            # constructed multi-GPU wrapper: the reference has no distributed mode, so the ranks' host gradients
            # are summed with NCCL through a device staging buffer between fwd_bwd and step
            torch.cuda.synchronize()        # the engine writes every layer's gradients back to the host on its own
            bufs = []                       # outbound stream at the end of that layer's backward: let those copies land
            b = am.buffers
            for d in (getattr(b, "host_grads", None) or []):
                bufs += list(d.values()) if isinstance(d, dict) else [d]
            for name in ("gpu_embed_grads", "gpu_head_grads"):        # device-resident dicts in the reference engine
                d = getattr(b, name, None)
                if isinstance(d, dict):
                    bufs += list(d.values())
            for t in bufs:
                g = t.to(dev, non_blocking=True) if not t.is_cuda else t
                dist.all_reduce(g)
                if not t.is_cuda:
                    t.copy_(g, non_blocking=True)
            torch.cuda.synchronize()

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def ref_loss(st):
            """Mean loss of the whole job's batch from the reference's StepStats (sum of per-token losses)."""
            t = torch.tensor([float(st.total_loss)], dtype=torch.float64, device=dev)
            if world > 1:
                dist.all_reduce(t)
            return float(t) / gbatch

        def agree(ok: bool) -> bool:
            """True only if every rank says so (the ranks must walk the plan ladder in lock-step)."""
            if world == 1:
                return ok
            t = torch.tensor([1 if ok else 0], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            return bool(int(t.item()))

        def worst_of(code: int) -> int:
            """Largest code over the ranks."""
            if world == 1:
                return code
            t = torch.tensor([code], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return int(t.item())

        def checked_step(seqs, sync: bool = False):
            """One optimisation step -> ``(StepStats, None)`` or ``(None, why)``.  The ranks tell one another whether
            they got through forward / backward before the gradient all-reduce, and through the optimizer step after
            it, so a rank whose engine raised (device memory, typically) never leaves the others in a collective."""
            failed, st = None, None
            try:
                st = am.fwd_bwd(seqs, loss_scale_factor=1.0 / gbatch, total_tokens_per_step=gbatch)
                if sync:
                    torch.cuda.synchronize()
            except Exception as e:
                failed = f"{type(e).__name__}: {str(e)[:160]}"
                del e
            if not agree(failed is None):
                return None, failed or "another rank failed in forward / backward"
            try:
                if world > 1:
                    allreduce_grads()
                am.step()
                if sync:
                    torch.cuda.synchronize()
            except Exception as e:
                failed = f"{type(e).__name__}: {str(e)[:160]}"
                del e
            if not agree(failed is None):
                return None, failed or "another rank failed in the optimizer step"
            return st, None

        def teardown(m) -> None:
            """Give back what a reference engine holds: its buffers and its cudaHostRegister'ed host memory (the
            reference's own process-wide clean-up, flextrain/engine/host_memory.py:215-233)."""
            import gc
            try:
                torch.cuda.synchronize()        # no copy of the engine may still be in flight on its side streams
            except Exception:
                pass
            try:
                b = getattr(m, "buffers", None)
                if b is not None and hasattr(b, "destroy"):
                    b.destroy()
            except Exception:
                pass
            try:
                from flextrain.engine import unregister_all_process_pinned_memory
                unregister_all_process_pinned_memory()
            except Exception:
                pass
            del m
            gc.collect()
            torch.cuda.empty_cache()

        am, errors, chosen = None, [], None
        # state dtype (the configuration's fp32 first, the reference's own bf16 default last) x GPU budget (descending:
        # the largest budget whose plan also survives the reference's own allocations wins) x link figure x chunk cap
        ladder = [(st, g, hw, m)
                  for st in ("float32", "bfloat16")
                  for g in (None, 150, 120, 96, 64, 31)
                  for hw in ("probed", "nominal")
                  for m in (None, 16384, 8192, 4096)]
        oom_at = set()                       # (state, gpu budget) whose plan ran out of device memory: skip its variants
        for st, g, hw, m in ladder:
            if (st, g) in oom_at:
                continue
            opt = AdamW(AdamWHyperparams(lr=3e-5, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0),
                        state_dtype=getattr(torch, st))
            hwc, mbw = hw_probed if hw == "probed" else hw_nominal
            try:
                am = ref.from_dims(dims, arch="llama", optimizer=opt, max_seq_len=seq_len,
                                   max_global_batch_tokens=per_rank,
                                   max_gpu_mem_bytes=int(free) if g is None else min(int(free), g << 30),
                                   max_host_mem_bytes=host_budget, max_chunk_size=m, hw_cost=hwc, mem_bw_gbps=mbw,
                                   hyperparams={"rope_theta": 500000.0, "rms_norm_eps": 1e-5}, device=dev)
                chosen = {"opt_state": st, "hw_cost": hw, "max_gpu_gib": g, "max_chunk_size": m}
            except Exception as e:        # whatever it is: the ranks must stay in lock-step (see agree below)
                msg = f"{st}/gpu={g}/{hw}/chunk={m}: {type(e).__name__}: {str(e)[:160]}"
                errors.append(msg)
                print("[reference arm] attempt failed: " + msg.replace("\n", " "), file=sys.stderr, flush=True)
                if len(errors) == 1 and rank == 0 and isinstance(e, ValueError):
                    # the planner's own trace of the first (preferred) attempt, so a log shows why it was refused
                    import contextlib
                    with contextlib.redirect_stdout(sys.stderr):
                        try:
                            ref.from_dims(dims, arch="llama", optimizer=opt, max_seq_len=seq_len,
                                          max_global_batch_tokens=per_rank, max_gpu_mem_bytes=int(free),
                                          max_host_mem_bytes=host_budget, max_chunk_size=m, hw_cost=hwc,
                                          mem_bw_gbps=mbw, device=dev, verbose=True,
                                          hyperparams={"rope_theta": 500000.0, "rms_norm_eps": 1e-5})
                        except Exception:
                            pass
                status = 1                  # refused by the planner
                if not isinstance(e, ValueError):
                    status = 2              # an allocation of the reference's own plan failed (device or pinned memory)
                    del e
                    teardown(None)          # also drops the host registrations of the half-built engine
                am = None
            else:
                status = 0
            worst = worst_of(status)
            if worst == 2:
                # on some rank: the other link / chunk variants of this budget plan the same memory, so every rank goes
                # to the next smaller GPU budget
                oom_at.add((st, g))
            if worst != 0:
                if am is not None:
                    errors.append(f"{st}/gpu={g}/{hw}/chunk={m}: built here, " +
                                  ("refused" if worst == 1 else "out of memory") + " on another rank")
                    teardown(am)
                    am = None
                continue
            # The plan built on every rank.  The warm-up steps are part of the attempt: a plan that takes the whole GPU
            # can still run out of device memory in the reference's own step-time allocations (seen at 8 ranks: round =
            # chunk = 65,536 tokens, 23 layers resident); then the engine is given back and the next smaller GPU budget
            # is planned.
            src = SyntheticTokenSource(dims["vocab_size"], seq_len, seed=1234)      # every attempt sees the same batches
            failed, st_first, warm_s = None, None, 0.0
            for i in range(args.warmup):
                barrier()
                t0 = time.perf_counter()
                st_i, failed = checked_step(next_batch(), sync=True)
                if failed is not None:
                    failed = f"warm-up step {i + 1}: {failed}"
                    break
                barrier()
                warm_s = time.perf_counter() - t0
                if i == 0:
                    st_first = st_i
            if failed is not None:
                msg = f"{st}/gpu={g}/{hw}/chunk={m}: {failed}"
                errors.append(msg)
                print("[reference arm] attempt failed: " + msg.replace("\n", " "), file=sys.stderr, flush=True)
                oom_at.add((st, g))
                st_i = st_first = None
                teardown(am)
                am = None
                continue
            break
        if am is None:
            for line in errors:
                print("[reference arm] " + line, file=sys.stderr)
            try:                                    # the planner's own trace for the last attempt
                ref.from_dims(dims, arch="llama", optimizer=opt, max_seq_len=seq_len, max_global_batch_tokens=per_rank,
                              max_gpu_mem_bytes=int(free), max_host_mem_bytes=host_budget, hw_cost=hw_probed[0],
                              mem_bw_gbps=hw_probed[1], device=dev, verbose=True,
                              hyperparams={"rope_theta": 500000.0, "rms_norm_eps": 1e-5})
            except Exception:
                pass
            raise RuntimeError(f"no plan builds ({len(errors)} attempts); first: {errors[0]}; last: {errors[-1]}")
        ws = am.working_set if hasattr(am, "working_set") else None
        if rank == 0:
            print(f"[reference arm] plan {chosen}: " + (f"round {ws.target_round_tokens} chunk {ws.max_chunk_size} "
                  f"gpu layers {ws.n_gpu_layers}/{ws.n_gpu_grads}/{ws.n_gpu_opt_layers} host act "
                  f"{ws.host_act_buffer_size / 2 ** 30:.1f} GiB" if ws is not None else ""), file=sys.stderr, flush=True)
        loss_step1 = ref_loss(st_first) if st_first is not None else None
        steps = _budget_steps(args, t_proc0, warm_s)
        if world > 1:
            tsteps = torch.tensor([steps], device=dev)
            dist.all_reduce(tsteps, op=dist.ReduceOp.MIN)
            steps = int(tsteps.item())
        sampler = ClockSampler(local)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for _ in range(steps):
            st, failed = checked_step(next_batch())
            if failed is not None:              # every rank is told, so all of them leave through the same door
                sampler.stop()
                raise RuntimeError(f"a timed step failed after {args.warmup} good warm-up steps: {failed}")
        e1.record()
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        dev_ms = e0.elapsed_time(e1)
        clocks = sampler.stop()
        t = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = float(t[0]), float(t[1])
        last_loss = ref_loss(st)
    except Exception as e:
        import traceback
        traceback.print_exc()
        unavailable(f"reference run failed on this box: {type(e).__name__}: {e}")
    if rank == 0:
        ms_step = dev_ms / steps
        value = gbatch / (ms_step / 1e3)
        _emit({"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world,
               "steps": steps, "steps_requested": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
               "higher_is_better": True,
               "scaling": "strong", "vs_baseline": value / PUBLISHED_TOK_S, "dtype": "bf16",
               "data": "synthetic uniform tokens, random-init weights",
               "config": {"model": "Llama-3.1-8B" + (" (SMALL DEBUG)" if args.small else ""), "global_batch": gbatch,
                          "seq_len": seq_len,
                          "parallelism": f"dp{world}" + (" (constructed: one reference engine per GPU + NCCL "
                                                         "all-reduce of host gradients)" if world > 1 else ""),
                          "optimizer": f"AdamW {chosen['opt_state']} state", "plan": chosen,
                          "round_tokens": getattr(ws, "target_round_tokens", None),
                          "chunk": getattr(ws, "max_chunk_size", None),
                          "gpu_layers": getattr(ws, "n_gpu_layers", None),
                          "host_budget_gib": host_budget / 2 ** 30},
               "clocks": clocks,
               "e2e": {"value": gbatch / (e2e_ms / steps / 1e3), "unit": "tokens/s",
                       "h2d_bytes_per_step": 16 * per_rank, "d2h_bytes_per_step": 4 * per_rank},
               "loss": last_loss, "loss_step1": loss_step1,
               "gpu_launches": None})
    if world > 1:
        dist.destroy_process_group()


def main():
    _claim_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--config", choices=sorted(CONFIGS), default="llama8b",
                    help="named configuration; the headline number is llama8b")
    ap.add_argument("--shard", default=None, help="data-parallel shard mode (default: planner's choice)")
    ap.add_argument("--chunk", type=int, default=None)
    ap.add_argument("--head-chunk", type=int, default=4096)
    ap.add_argument("--host-gib", type=int, default=64)
    ap.add_argument("--budget-s", type=float, default=800.0,
                    help="wall-clock budget of the whole process; timed steps are reduced to fit (0 = never)")
    ap.add_argument("--opt-state-device", action="store_true",
                    help="keep optimizer state in HBM even for a configuration that names host offload (llama70b)")
    ap.add_argument("--op-timing", default=None, metavar="FILE",
                    help="bracket every op with CUDA events and write the per-op time table of the timed steps to FILE "
                         "(diagnostic run: the throughput it prints is not a benchmark value)")
    ap.add_argument("--small", action="store_true", help="4-layer debug model; results are not reportable")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
