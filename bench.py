"""Headline benchmark: trained tokens/s for the whole job, Llama-3.1-8B full fine-tune.

    python bench.py --gpus 1 --steps 2 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W
    python bench.py --impl reference ...          # the unmodified reference engine, same metric and config

Config (fixed): 32 layers, hidden 4096, 32 query / 8 KV heads, head_dim 128, SwiGLU 14336, vocab 128256, RoPE
theta 5e5; bf16 weights / activations / gradients, fp32 AdamW state; synthetic uniform tokens, seq_len 1024,
global batch 524288 tokens per optimizer step (strong scaling: the global batch is split over the GPUs);
random-init weights.  Every timed step runs forward, backward, the data-parallel gradient reduction and the
optimizer update.  Two timed regions of K steps each, after W warm-up steps:
  * device-timed (CUDA events on the compute stream, max over ranks) -> ``value``;
  * end to end (wall clock around the public API: host token generation into pinned memory, H2D copy of the
    step's tokens, ``fwd_bwd`` + ``step``, D2H read of the loss) -> ``e2e``.
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
                    hyper={"rope_theta": 500000.0, "norm_eps": 1e-5}, scaling="strong"),
    # long-context dense 12B: one 32768-token sequence per GPU (weak scaling), chunked attention with a KV window
    "longctx12b": dict(model="dense-12B long context", arch="llama",
                       dims=dict(vocab_size=131072, n_layers=40, d_model=5120, n_heads=32, n_kv_heads=8, head_dim=128,
                                 expert_dim=14336, ffn_dim=14336, num_routed_experts=0, num_shared_experts=0, top_k=0,
                                 is_causal=True),
                       seq_len=32768, per_gpu_batch=32768, hyper={"rope_theta": 1000000.0, "norm_eps": 1e-5},
                       scaling="weak"),
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
                     scaling="strong", tp="world"),
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


def _emit(obj):
    print(json.dumps(obj), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist

    import flextrain_b200 as ft
    from flextrain_b200 import ops
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
    per_rank = gbatch if par["tp"] > 1 else gbatch // world
    free, total = torch.cuda.mem_get_info()
    opt = ft.AdamW(lr=3e-5, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, state_dtype=torch.float32)
    am = ft.from_dims(dims, arch=cfg["arch"], optimizer=opt, max_seq_len=seq_len, max_global_batch_tokens=gbatch,
                      max_gpu_mem_bytes=int(free), max_host_mem_bytes=args.host_gib << 30, device=dev,
                      hyperparams=cfg["hyper"], world_size=world, rank=rank,
                      dp_shard=args.shard, init_on_device=True, init_std=0.02, verbose=(rank == 0 and args.verbose),
                      max_chunk_size=args.chunk, head_chunk_size=args.head_chunk, **par)
    src = ft.SyntheticTokenSource(dims["vocab_size"], seq_len, seed=1234 + (0 if par["tp"] > 1 else rank), pin=True)

    def one_step(seqs):
        st = am.fwd_bwd(seqs, loss_scale_factor=1.0 / gbatch, total_tokens_per_step=gbatch)
        rc = am.step()
        assert rc == 0
        return st

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        st = one_step(src.get_sequences(per_rank))
    barrier()
    peak_alloc = torch.cuda.max_memory_allocated() / 2 ** 30

    # ---- region A: device-timed
    batches = [src.get_sequences(per_rank) for _ in range(args.steps)]
    sampler = ClockSampler(local)
    ops.reset_launch_count()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for seqs in batches:
        st = one_step(seqs)
    e1.record()
    barrier()
    dev_ms = e0.elapsed_time(e1)
    launches = ops.launch_count()
    clocks = sampler.stop()
    last_loss = st.loss
    # ---- region B: end to end through the public API
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        seqs = src.get_sequences(per_rank)             # host RNG into pinned memory
        st = one_step(seqs)                            # H2D of tokens/targets, fwd+bwd+step, D2H of the loss
    barrier()
    e2e_s = time.perf_counter() - t0

    t = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = float(t[0]), float(t[1])
    errs = kernels.device_error_words()
    if rank == 0:
        ms_step = dev_ms / args.steps
        value = gbatch / (ms_step / 1e3)
        e2e_val = gbatch / (e2e_ms / args.steps / 1e3)
        n_params = 0
        for scope, l, name, t in am.named_master_params():
            sp = am.spec_of(scope, l, name)
            if sp.shard.ep_dim is not None:       # routed experts: only top_k of num_experts are active per token
                n_params += t.numel() * par["ep"] * dims["top_k"] // dims["num_routed_experts"]
            else:
                n_params += t.numel() * (par["tp"] if sp.is_local_part else 1)
        flops_tok = 6.0 * (n_params - dims["vocab_size"] * dims["d_model"]) \
            + 6.0 * seq_len * dims["n_heads"] * dims["head_dim"] * dims["n_layers"]
        tflops_gpu = value * flops_tok / world / 1e12
        peaks = {}
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                peaks = json.load(f)
        except Exception:
            pass
        sustained = peaks.get("bf16_tflops_sustained", 1400.0)
        _emit({
            "metric": METRIC if args.config == "llama8b" else f"train tokens/sec/box, {cfg['model']} full FT",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": cfg["scaling"],
            "vs_baseline": value / PUBLISHED_TOK_S if args.config == "llama8b" else None, "dtype": "bf16", "data": "synthetic uniform tokens, random-init weights",
            "config": {"model": cfg["model"] + (" (SMALL DEBUG)" if args.small else ""), "global_batch": gbatch,
                       "seq_len": seq_len, "parallelism": (f"tp{world}" if par["tp"] > 1 else f"dp{world}" + (f"+ep{world}" if par["ep"] > 1 else ""))
                       + (f"-shard({am.ws.shard})" if world > 1 else ""),
                       "optimizer": "AdamW fp32 state", "round_tokens": am.ws.target_round_tokens,
                       "chunk": am.ws.max_chunk_size, "rounds_per_step": am.ws.target_num_rounds,
                       "l2": "inputs larger than L2 (each step streams >100 GB of weights/activations)",
                       "gemm_backend": os.environ.get("FTB_GEMM_BACKEND", "tcgen05"),
                       "attention_backend": ops.get_attention_backend()},
            "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": "tokens/s", "h2d_bytes_per_step": 16 * per_rank,
                    "d2h_bytes_per_step": 4 * per_rank + 12},
            "gpu_launches": launches,
            "model_tflops_per_gpu": tflops_gpu, "pct_of_measured_sustained_bf16": 100.0 * tflops_gpu / sustained,
            "loss": last_loss, "peak_alloc_gib": peak_alloc, "device_errors": errs,
        })
    if world > 1:
        dist.destroy_process_group()


def run_reference(args):
    """The unmodified reference engine (installed under baseline/_ref) through its own public API."""
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
        dev = f"cuda:{local}"
        if world > 1:
            dist.init_process_group("nccl", device_id=torch.device(dev))
        import flextrain as ref
        from flextrain.io.sources import SyntheticTokenSource
        from flextrain.optim.adamw import AdamW, AdamWHyperparams
    except Exception as e:
        unavailable(f"reference import failed: {type(e).__name__}: {e}")
    try:
        import psutil
        dims = {k: v for k, v in LLAMA31_8B.items() if k != "ffn_dim"}
        seq_len, gbatch = SEQ_LEN, GLOBAL_BATCH
        if args.small:
            dims["n_layers"] = 4
            gbatch = 65536
        per_rank = gbatch // world
        free, _ = torch.cuda.mem_get_info()
        host_free = int(psutil.virtual_memory().available * 0.8) // max(world, 1)
        opt = AdamW(AdamWHyperparams(lr=3e-5, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0),
                    state_dtype=torch.float32)
        # The reference planner can reject its default chunk candidates on a 180 GB GPU and then advises a smaller
        # --max-chunk-size; follow that advice through the public keyword until a plan exists.
        am, plan_err = None, None
        for mcs in (None, 16384, 8192, 4096):
            try:
                am = ref.from_dims(dims, arch="llama", optimizer=opt, max_seq_len=seq_len,
                                   max_global_batch_tokens=per_rank, max_gpu_mem_bytes=int(free),
                                   max_host_mem_bytes=host_free, max_chunk_size=mcs,
                                   hyperparams={"rope_theta": 500000.0, "rms_norm_eps": 1e-5}, device=dev)
                ref_chunk = mcs
                break
            except ValueError as e:
                plan_err = e
        if am is None:
            raise plan_err
        src = SyntheticTokenSource(dims["vocab_size"], seq_len, seed=1234 + rank)

        def allreduce_grads():
            # constructed multi-GPU wrapper: the reference has no distributed mode, so the ranks' host gradients
            # are summed with NCCL through a device staging buffer between fwd_bwd and step
            bufs = []
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

        def one_step(seqs):
            st = am.fwd_bwd(seqs, loss_scale_factor=1.0 / gbatch, total_tokens_per_step=gbatch)
            if world > 1:
                allreduce_grads()
            am.step()
            return st

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        for _ in range(args.warmup):
            one_step(src.get_sequences(per_rank))
        barrier()
        batches = [src.get_sequences(per_rank) for _ in range(args.steps)]
        sampler = ClockSampler(local)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for seqs in batches:
            st = one_step(seqs)
        e1.record()
        barrier()
        dev_ms = e0.elapsed_time(e1)
        clocks = sampler.stop()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            st = one_step(src.get_sequences(per_rank))
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
        t = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, e2e_ms = float(t[0]), float(t[1])
    except Exception as e:
        import traceback
        traceback.print_exc()
        unavailable(f"reference run failed on this box: {type(e).__name__}: {e}")
    if rank == 0:
        ms_step = dev_ms / args.steps
        value = gbatch / (ms_step / 1e3)
        _emit({"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world,
               "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
               "scaling": "strong", "vs_baseline": value / PUBLISHED_TOK_S, "dtype": "bf16",
               "data": "synthetic uniform tokens, random-init weights",
               "config": {"model": "Llama-3.1-8B" + (" (SMALL DEBUG)" if args.small else ""), "global_batch": gbatch,
                          "seq_len": seq_len,
                          "parallelism": f"dp{world}" + (" (constructed: one reference engine per GPU + NCCL "
                                                         "all-reduce of host gradients)" if world > 1 else "")},
               "clocks": clocks,
               "e2e": {"value": gbatch / (e2e_ms / args.steps / 1e3), "unit": "tokens/s",
                       "h2d_bytes_per_step": 16 * per_rank, "d2h_bytes_per_step": 4 * per_rank},
               "gpu_launches": None})
    if world > 1:
        dist.destroy_process_group()


def main():
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
    ap.add_argument("--small", action="store_true", help="4-layer debug model; results are not reportable")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
