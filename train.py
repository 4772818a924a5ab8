"""End-to-end training CLI (same flags as the reference's train.py:372-630, plus the parallel layout).

    python train.py --model <hf dir | dims:<name>> --mode {full,lora} --max-seq-len N --max-global-batch-tokens N
    python -m torch.distributed.run --nproc-per-node 8 train.py ... --dp-shard opt+grad

Per step: LR schedule (linear warm-up → constant → cosine to ``final``), ``source.get_sequences``, the
short-tail-round spill (sequences that would open an extra, nearly empty round go back to the source),
``am.fwd_bwd`` + ``am.step``, and a log line with loss / tok/s / effective and hardware TFLOPS / memory.
``--save`` writes ``final.safetensors`` in HF names.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import flextrain_b200 as ft  # noqa: E402
from flextrain_b200.core.flop_accounting import step_flops_breakdown  # noqa: E402
from flextrain_b200.core._memory import get_available_gpu_memory, get_available_host_memory  # noqa: E402
from flextrain_b200.engine.schedule import split_sequences  # noqa: E402

_DT = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


def lr_schedule(step: int, *, max_lr: float, final_lr: float, warmup_steps: int, cooldown_start: int,
                total_steps: int) -> float:
    """``step`` is 1-based. Linear warm-up ``max*step/warmup`` → ``max`` → cosine to ``final`` from ``cooldown_start``."""
    if warmup_steps > 0 and step <= warmup_steps:
        return max_lr * step / warmup_steps
    if step <= cooldown_start or total_steps <= cooldown_start:
        return max_lr
    t = (step - cooldown_start) / max(1, total_steps - cooldown_start)
    return final_lr + 0.5 * (max_lr - final_lr) * (1 + math.cos(math.pi * min(t, 1.0)))


def build_arg_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="train.py")
    p.add_argument("--model", required=True, help="HF model directory, or dims:<name> (a random-init catalogue model) / dims:<file.json> (a dims dict)")
    p.add_argument("--mode", choices=("full", "lora"), required=True)
    p.add_argument("--max-seq-len", type=int, required=True)
    p.add_argument("--max-global-batch-tokens", type=int, required=True)
    p.add_argument("--truncate-long", action="store_true")
    p.add_argument("--apply-chat-template", action="store_true")
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--data-source", choices=("json_sft", "synthetic", "shards", "mm_json", "hf", "raw", "custom"),
                   default="json_sft",
                   help="mm_json: chat rows with image / video files for a vision-language checkpoint; hf: a HuggingFace "
                        "`datasets` id or directory in --dataset; raw: a .pt file of pre-tokenised sequences; custom: "
                        "--custom-factory module:callable returning (records, extract)")
    p.add_argument("--train-vision-tower", action="store_true",
                   help="vision-language checkpoints: update the vision tower too (default: frozen)")
    p.add_argument("--tokenizer", default=None, help="tokenizer directory / hub id (default: the model directory)")
    p.add_argument("--min-seq-len", type=int, default=0, help="skip documents / records shorter than this")
    p.add_argument("--hf-subset", default=None)
    p.add_argument("--hf-split", default="train")
    p.add_argument("--hf-text-field", default="text")
    p.add_argument("--no-hf-streaming", action="store_true")
    p.add_argument("--shard-documents", action="store_true",
                   help="shards: one sequence per document (split at the end-of-text id) instead of fixed windows")
    p.add_argument("--shard-num-shards", type=int, default=None)
    p.add_argument("--sft-prompt-field", default="instruction")
    p.add_argument("--sft-response-field", default="output")
    p.add_argument("--sft-input-field", default="input")
    p.add_argument("--custom-factory", default=None, metavar="MODULE:CALLABLE")
    p.add_argument("--dataset", default=os.path.join(ROOT, "flextrain_b200/configs/examples/data/tiny_math_sft.json"))
    p.add_argument("--synthetic-seq-len", type=int, default=None)
    p.add_argument("--output-dir", default=None)
    p.add_argument("--lr", type=float, default=None)
    p.add_argument("--lr-warmup-pct", type=float, default=0.1)
    p.add_argument("--lr-cooldown-start-pct", type=float, default=0.8)
    p.add_argument("--lr-final-pct", type=float, default=0.1)
    p.add_argument("--lora-rank", type=int, default=16)
    p.add_argument("--lora-alpha", type=float, default=16.0)
    p.add_argument("--attn-backend", default="auto", choices=["auto", "ftb", "library", "eager"],
                   help="ftb: the hand-written sm_100a kernels (what auto picks on a B200); library: torch's bundled "
                        "flash kernels (comparison only); eager: plain PyTorch")
    p.add_argument("--use-muon", action="store_true")
    p.add_argument("--device-id", type=int, default=None)
    p.add_argument("--max-gpu-mem-gib", type=float, default=None)
    p.add_argument("--max-host-mem-gib", type=float, default=None)
    p.add_argument("--leeway-gpu-mem-gib", type=float, default=5.0)
    p.add_argument("--leeway-host-mem-gib", type=float, default=10.0)
    p.add_argument("--profile-start-step", type=int, default=None)
    p.add_argument("--profile-stop-step", type=int, default=None)
    p.add_argument("--force-save-level", type=int, default=None, choices=[0, 1, 2, 3])
    p.add_argument("--min-chunk-size", type=int, default=None)
    p.add_argument("--max-chunk-size", type=int, default=None)
    p.add_argument("--master-dtype", choices=tuple(_DT), default="bfloat16")
    p.add_argument("--grad-dtype", choices=tuple(_DT), default="bfloat16")
    p.add_argument("--opt-state-dtype", choices=tuple(_DT), default=None)
    p.add_argument("--opt-state", choices=("auto", "host", "device"), default="auto",
                   help="where optimizer state lives: the planner decides, pinned host memory (streamed through a "
                        "device ring during the step), or HBM")
    p.add_argument("--save", action="store_true")
    p.add_argument("--save-state-every", type=int, default=0,
                   help="every N steps (and at the end) write a full training state (weights, optimizer state, step) "
                        "to <output-dir>/state; 0 = never")
    p.add_argument("--max-grad-norm", type=float, default=None,
                   help="clip the global gradient norm to this value before every update (library-collective or "
                        "single-GPU runs; the norm is logged as gnorm)")
    p.add_argument("--eval-every", type=int, default=0, help="every N steps: validation loss (forward only); 0 = never")
    p.add_argument("--eval-dataset", default=None, help="validation file(s), same kind as --dataset")
    p.add_argument("--eval-tokens", type=int, default=65536, help="validation tokens per evaluation, over all ranks")
    p.add_argument("--metrics-jsonl", default=None,
                   help="append one JSON object per step (rank 0): step, loss, ema, lr, tokens, tok/s, TFLOPS, memory, "
                        "rounds / chunks, save-tier histogram; default <output-dir>/metrics.jsonl, 'none' disables")
    p.add_argument("--stop-after", type=int, default=None,
                   help="leave the loop after this step (the schedule still spans --steps): a run that will be resumed")
    p.add_argument("--resume-state", default=None,
                   help="directory written by --save-state-every: restore it and continue from its step (same model, "
                        "world size and layout; the data source is advanced past the batches already consumed)")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--verbose", action="store_true")
    # parallel layout (new): ranks come from torch.distributed.run
    p.add_argument("--dp-shard", default=None, choices=["opt+grad", "opt+grad+param"])
    p.add_argument("--heartbeat-s", type=float, default=0.0,
                   help="multi-rank runs: raise on every rank when a peer has not finished a step for this many "
                        "seconds or has left (0 = off)")
    _deg = lambda v: v if v == "auto" else int(v)
    p.add_argument("--tp", type=_deg, default=1, help="tensor-parallel degree, or 'auto': plan data / expert / tensor "
                   "parallel layouts for this model and budget and take the fastest that fits")
    p.add_argument("--ep", type=_deg, default=1, help="expert-parallel degree, or 'auto' (see --tp)")
    return p


def _attn_backend(name: str) -> str:
    return name


def _resolve_model(args):
    if args.model.startswith("dims:"):
        with open(os.path.join(ROOT, "flextrain_b200/configs/model_dims.json")) as f:
            cat = json.load(f)
        name = args.model[5:]
        if name.endswith(".json") and os.path.exists(name):        # {"arch": ..., "hyperparams": {...}, <dims keys>}
            with open(name) as f:
                return "dims", json.load(f)
        if name not in cat:
            raise SystemExit(f"unknown dims model {name!r}; known: {sorted(cat)}")
        return "dims", cat[name]
    if not os.path.isdir(args.model):
        from flextrain_b200.io.download import maybe_download_hf_snapshot
        args.model = maybe_download_hf_snapshot(args.model, os.environ.get("FLEXTRAIN_MODELS_DIR", "models"))
    return "hf", args.model


def main(argv=None) -> int:
    args = build_arg_parser().parse_args(argv)
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available()
    dev_id = args.device_id if args.device_id is not None else local
    device = f"cuda:{dev_id}" if use_cuda else "cpu"
    if use_cuda:
        torch.cuda.set_device(dev_id)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl" if use_cuda else "gloo",
                                **({"device_id": torch.device(device)} if use_cuda else {}))
    say = print if rank == 0 else (lambda *a, **k: None)
    ft_ops = __import__("flextrain_b200.ops", fromlist=["set_attention_backend"])
    ft_ops.set_attention_backend(_attn_backend(args.attn_backend))

    # ---- optimizer (flextrain train.py:677-720)
    lora = args.mode == "lora"
    sd = _DT[args.opt_state_dtype] if args.opt_state_dtype else (torch.float32 if lora else torch.bfloat16)
    if lora:
        if args.use_muon:
            raise SystemExit("--use-muon is for full fine-tuning only")
        opt = ft.AdamW(lr=args.lr or 1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, state_dtype=sd)
    elif args.use_muon:
        lr = args.lr or 1e-3
        opt = ft.HybridMuonAdamW(muon=ft.Muon(lr=lr), adamw=ft.AdamW(lr=lr, state_dtype=sd))
    else:
        opt = ft.AdamW(lr=args.lr or 3e-5, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0, state_dtype=sd)

    # ---- budgets
    gpu_b = int(args.max_gpu_mem_gib * 2 ** 30) if args.max_gpu_mem_gib else get_available_gpu_memory(device)
    env_cap = os.environ.get("FLEXTRAIN_MAX_GPU_MEM_GIB")
    if env_cap:
        gpu_b = min(gpu_b, int(float(env_cap) * 2 ** 30))
    host_b = int(args.max_host_mem_gib * 2 ** 30) if args.max_host_mem_gib else get_available_host_memory() // max(world, 1)
    say(f"[budget] gpu {gpu_b / 2**30:.1f} GiB, host {host_b / 2**30:.1f} GiB, world {world}")

    kind, model = _resolve_model(args)
    common = dict(optimizer=opt, max_seq_len=args.max_seq_len, max_global_batch_tokens=args.max_global_batch_tokens,
                  max_gpu_mem_bytes=gpu_b, max_host_mem_bytes=host_b, device=device,
                  leeway_gpu_mem_bytes=int(args.leeway_gpu_mem_gib * 2 ** 30),
                  leeway_host_mem_bytes=int(args.leeway_host_mem_gib * 2 ** 30),
                  compute_dtype=torch.bfloat16 if use_cuda else torch.float32,
                  master_dtype=_DT[args.master_dtype] if use_cuda else torch.float32,
                  grad_dtype=_DT[args.grad_dtype] if use_cuda else torch.float32,
                  lora_targets="all" if lora else None, lora_rank=args.lora_rank, lora_alpha=args.lora_alpha,
                  force_saved_act_level=args.force_save_level, min_chunk_size=args.min_chunk_size,
                  max_chunk_size=args.max_chunk_size, verbose=args.verbose and rank == 0, world_size=world, rank=rank,
                  dp_shard=args.dp_shard, tp=args.tp, ep=args.ep, opt_state=args.opt_state)
    if kind == "dims":
        arch = model.pop("arch", "llama")
        hyper = model.pop("hyperparams", None)
        am = ft.from_dims(model, arch=arch, hyperparams=hyper, init_on_device=use_cuda, **common)
        vocab = model["vocab_size"]
    else:
        am = ft.from_pretrained(model, freeze_modality_encoders=not args.train_vision_tower, **common)
        if os.environ.get("FLEXTRAIN_RANDOMIZE_WEIGHTS") == "1":
            from flextrain_b200.api import _init_random_weights
            _init_random_weights(am, int(os.environ.get("FLEXTRAIN_RANDOMIZE_WEIGHTS_SEED", "0")),
                                 float(os.environ.get("FLEXTRAIN_RANDOMIZE_WEIGHTS_STD", "0.02")), on_device=use_cuda)
        vocab = am.model_config.vocab_size

    # ---- data
    # data-parallel ranks (also under expert parallelism) each take their share of the batch; the ranks of a
    # tensor-parallel group work on the SAME sequences, so they read identical data
    tp_deg = getattr(am, "tp_degree", args.tp)
    data_ranks, data_rank = (world // tp_deg, rank // tp_deg) if tp_deg > 1 else (world, rank)
    per_rank_tokens = args.max_global_batch_tokens // data_ranks
    def make_source(path, seed, loop=True):
        if args.data_source == "synthetic":
            return ft.SyntheticTokenSource(vocab, args.synthetic_seq_len or args.max_seq_len, seed=seed + data_rank,
                                           pin=use_cuda)
        def tokenizer():
            from transformers import AutoTokenizer
            return AutoTokenizer.from_pretrained(args.tokenizer or (model if kind == "hf" else args.model))

        if args.data_source == "shards":
            if args.shard_documents:
                s = ft.ShardTokenSource(path, loop=loop, vocab_size=vocab, num_shards=args.shard_num_shards,
                                        min_seq_len=args.min_seq_len, max_seq_len=args.max_seq_len)
            else:
                s = ft.ShardTokenSource(path, args.max_seq_len, loop=loop, num_shards=args.shard_num_shards)
        elif args.data_source == "hf":
            s = ft.HFTokenSource(path, tokenizer(), subset=args.hf_subset, split=args.hf_split,
                                 text_field=args.hf_text_field, min_seq_len=args.min_seq_len,
                                 max_seq_len=args.max_seq_len, streaming=not args.no_hf_streaming)
        elif args.data_source == "raw":
            s = ft.RawTokenSource(torch.load(path, map_location="cpu"), loop=loop)
        elif args.data_source == "custom":
            import importlib
            mod_name, _, attr = (args.custom_factory or "").partition(":")
            if not attr:
                raise SystemExit("--data-source custom needs --custom-factory module:callable")
            records, extract = getattr(importlib.import_module(mod_name), attr)()
            s = ft.CustomSchemaTokenSource(records, extract, loop=loop)
        elif args.data_source == "mm_json":
            if kind != "hf":
                raise SystemExit("--data-source mm_json needs an HF vision-language model directory (tokenizer, geometry)")
            from flextrain_b200.io.image_processing import MultimodalProcessorBundle
            s = ft.MultimodalJsonSource(path, MultimodalProcessorBundle.from_pretrained(model), args.max_seq_len, loop=loop)
        else:
            s = ft.JsonSFTTokenSource(path, tokenizer(), args.max_seq_len, apply_chat_template=args.apply_chat_template,
                                      truncate_long=args.truncate_long, loop=loop, prompt_field=args.sft_prompt_field,
                                      response_field=args.sft_response_field, input_field=args.sft_input_field,
                                      min_seq_len=args.min_seq_len)
        # every rank opened the same files: data-parallel ranks each take every data_ranks-th sequence
        return ft.RankStridedSource(s, data_rank, data_ranks) if data_ranks > 1 else s

    src = make_source(args.dataset, args.seed)
    args._eval = None
    if args.eval_every > 0:
        if args.data_source != "synthetic" and not args.eval_dataset:
            raise SystemExit("--eval-every needs --eval-dataset (except with synthetic data)")
        args._eval = lambda: make_source(args.eval_dataset, args.seed + 7919, loop=False)
    out_dir = args.output_dir or os.path.join("runs", f"{os.path.basename(str(args.model).rstrip('/'))}_{args.mode}_sl{args.max_seq_len}")
    os.makedirs(out_dir, exist_ok=True)
    first_step = 1
    if args.resume_state:
        info = am.load_training_state(args.resume_state)
        first_step = info["step"] + 1
        for _ in range(info["step"]):                          # the batches the saved run already consumed
            src.get_sequences(per_rank_tokens)
        say(f"[resume] {args.resume_state}: continuing at step {first_step}")
    args._first_step, args._state_dir = first_step, os.path.join(out_dir, "state")
    mj = args.metrics_jsonl or os.path.join(out_dir, "metrics.jsonl")
    args._metrics_path = None if (rank != 0 or str(mj).lower() == "none") else mj
    rc = run_training_loop(am, src, args, per_rank_tokens, world, say)
    if args.save and (rank == 0 or am.tp is not None or am.ep is not None):
        # gathering tensor- / expert-parallel parts is a collective: every rank takes part, rank 0 writes
        path = am.save_hf(out_dir, "final.safetensors")
        say(f"[save] {path}")
        if args.mode == "lora":
            # final.safetensors holds the (frozen) base weights; what was trained is the adapter
            from flextrain_b200.export import save_lora_adapter
            apath = save_lora_adapter(am, os.path.join(out_dir, "adapter"),
                                      base_model_name_or_path=str(args.model))
            say(f"[save] {apath}")
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return rc


def validation_loss(am, source, rank_tokens: int, batch_tokens: int, world: int):
    """Mean loss over up to ``rank_tokens`` tokens of this rank's share of ``source`` (forward only), averaged over the
    job; every rank runs the same number of evaluation batches so that collectives inside the model stay matched."""
    import torch
    n_batches = max(1, -(-rank_tokens // batch_tokens))
    tot, cnt = 0.0, 0
    for _ in range(n_batches):
        seqs = source.get_sequences(min(batch_tokens, rank_tokens))
        if am.tp is None and am.ep is None and not seqs:
            break
        if not seqs:
            raise RuntimeError("the validation set ran out on this rank while model-parallel peers still evaluate; "
                               "use a larger --eval-dataset or fewer --eval-tokens")
        st = am.evaluate(seqs)
        tot += st.loss_sum
        cnt += st.active_tokens
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([tot, float(cnt)], dtype=torch.float64 if am.device.type == "cpu" else torch.float32,
                         device=am.device)
        dist.all_reduce(t)
        tot, cnt = float(t[0]), int(t[1])      # tensor-parallel peers each scored (and counted) their token shard
    return tot / max(cnt, 1), cnt


def run_training_loop(am, src, args, per_rank_tokens: int, world: int, say) -> int:
    total = args.steps
    warm, cool = int(total * args.lr_warmup_pct), int(total * args.lr_cooldown_start_pct)
    max_lr = am.optimizer.lr
    final_lr = max_lr * args.lr_final_pct
    ws = am.ws
    ema, t_start, tok_total = None, time.time(), 0
    profiling = False
    hb = None
    if world > 1 and getattr(args, "heartbeat_s", 0) > 0:
        # ranks learn of a lost peer on the host, between steps, instead of inside a kernel's bounded wait
        import torch.distributed as dist
        from flextrain_b200.parallel.health import Heartbeat
        hb = Heartbeat(dist.distributed_c10d._get_default_store(), dist.get_rank(), world, stale_s=args.heartbeat_s)
        hb.beat(0)
    first = getattr(args, "_first_step", 1)
    if hb is not None and first > 1:
        hb.beat(first - 1)
    last = min(total, args.stop_after) if getattr(args, "stop_after", None) else total
    for step in range(first, last + 1):
        if hb is not None:
            hb.check(grace_s=args.heartbeat_s)
        am.optimizer.lr = lr_schedule(step, max_lr=max_lr, final_lr=final_lr, warmup_steps=warm, cooldown_start=cool,
                                      total_steps=total)
        seqs = src.get_sequences(per_rank_tokens)
        if not seqs:
            say(f"[step {step}] data source exhausted")
            break
        # short-tail-round spill (flextrain train.py:221-250)
        for _ in range(4):
            rounds = split_sequences(seqs, target_round_tokens=ws.target_round_tokens, max_chunk_size=ws.max_chunk_size,
                                     max_training_chunks=ws.max_training_chunks,
                                     max_total_round_tokens=ws.max_total_round_tokens)
            if len(rounds) <= ws.target_num_rounds or len(rounds[-1]) >= len(seqs):
                break
            src.push_back(rounds[-1])
            seqs = seqs[: -len(rounds[-1])]
        if args.profile_start_step is not None and step == args.profile_start_step and torch.cuda.is_available():
            torch.cuda.synchronize(); torch.cuda.profiler.start(); profiling = True
        step_tokens = sum(len(s) for s in seqs)
        active = max(1, sum(s.active_token_count for s in seqs))
        shared_batch = am.tp is not None                      # the ranks of a tensor-parallel group hold one batch
        group_size = am.tp.world if shared_batch else 1
        if world > group_size:
            import torch.distributed as dist
            t = torch.tensor([step_tokens, active], device=am.device, dtype=torch.int64)
            dist.all_reduce(t)                                # every member of a group reports the group's batch
            g_tokens, g_active = int(t[0]) // group_size, int(t[1]) // group_size
        else:
            g_tokens, g_active = step_tokens, active
        t0 = time.time()
        st = am.fwd_bwd(seqs, loss_scale_factor=1.0 / g_active, total_tokens_per_step=g_tokens)
        rc = am.step(max_grad_norm=args.max_grad_norm) if getattr(args, "max_grad_norm", None) else am.step()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        # a bounded device-side wait that ran out means this step used incomplete data: stop, do not train on it
        am.check_health()
        dt = time.time() - t0
        if hb is not None:
            hb.beat(step)
        stop = args.profile_stop_step if args.profile_stop_step is not None else (
            args.profile_start_step + 2 if args.profile_start_step is not None else None)
        if profiling and stop is not None and step == stop:
            torch.cuda.profiler.stop(); profiling = False
        if rc != 0:
            say(f"[step {step}] optimizer reported non-finite gradients (code {rc}); update skipped")
        loss_sum = st.loss_sum
        if shared_batch:                                      # each rank scored its token shard of the same batch
            import torch.distributed as dist
            t = torch.tensor([loss_sum], device=am.device, dtype=torch.float64 if am.device.type == "cpu" else torch.float32)
            dist.all_reduce(t, group=am.tp.pg)
            loss_sum = float(t)
        loss = loss_sum / max(active, 1)
        ema = loss if ema is None else 0.95 * ema + 0.05 * loss
        eff, hw = step_flops_breakdown(am, st, mode=args.mode)
        tok_total += g_tokens
        mem = (torch.cuda.max_memory_allocated() / 2 ** 30, torch.cuda.max_memory_reserved() / 2 ** 30) \
            if torch.cuda.is_available() else (0.0, 0.0)
        say(f"[step {step:4d}] lr {am.optimizer.lr:.3e} loss {loss:.4f} ema {ema:.4f} tok/step {g_tokens} "
            f"tok/s {g_tokens / dt:,.0f} TFLOPS_eff {eff * world / dt / 1e12:.1f} TFLOPS_hw {hw * world / dt / 1e12:.1f} "
            f"max_alloc {mem[0]:.1f} GiB max_reserve {mem[1]:.1f} GiB step {dt * 1e3:.0f} ms "
            f"elapsed {time.time() - t_start:.0f}s"
            + (f" gnorm {am.last_grad_norm:.4f}" if getattr(args, "max_grad_norm", None) else ""))
        mj = getattr(args, "_metrics_path", None)
        if mj:
            with open(mj, "a") as f:
                f.write(json.dumps({"step": step, "loss": loss, "ema": ema, "lr": am.optimizer.lr, "tokens": g_tokens,
                                    "tokens_total": tok_total, "tok_per_s": g_tokens / dt, "step_ms": dt * 1e3,
                                    "tflops_eff": eff * world / dt / 1e12, "tflops_hw": hw * world / dt / 1e12,
                                    "max_alloc_gib": mem[0], "max_reserved_gib": mem[1], "rounds": st.n_rounds,
                                    "chunks": st.n_chunks, "save_tiers": {str(k): v for k, v in st.plan_hist.items()},
                                    "host_act_bytes": st.host_act_bytes, "optimizer_rc": rc,
                                    "grad_norm": am.last_grad_norm if getattr(args, "max_grad_norm", None) else None,
                                    "wall_s": time.time() - t_start}) + "\n")
        if getattr(args, "_eval", None) is not None and (step % args.eval_every == 0 or step == last):
            vl, vn = validation_loss(am, args._eval(), args.eval_tokens // max(world // (am.tp.world if am.tp else 1), 1),
                                     per_rank_tokens, world)
            say(f"[eval {step:4d}] loss {vl:.4f} over {vn} tokens")
            if mj:
                with open(mj, "a") as f:
                    f.write(json.dumps({"step": step, "eval_loss": vl, "eval_tokens": vn}) + "\n")
        every = getattr(args, "save_state_every", 0)
        if every and (step % every == 0 or step == last):
            am.save_training_state(args._state_dir, extra={"tokens_seen": tok_total, "ema": ema})
            say(f"[state] step {step} -> {args._state_dir}")
    say(f"[done] {tok_total} tokens in {time.time() - t_start:.1f}s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
