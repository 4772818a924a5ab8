"""Random-init pretraining on FineWeb-format token shards with a token or FLOP budget and periodic evaluation
(flextrain/scripts/pretrain.py:1-44, 110-160, 518-571).

Two ways to name the model::

    python -m flextrain_b200 pretrain --arch llama --d-model 768 --n-layers 12 --vocab-size 50304 \\
        --total-tokens 1B --batch-tokens 16384 --data-dir /data/fineweb10B --train-shards 1-99 --val-shard 0 \\
        --out runs/llama_124M_1B
    python -m flextrain_b200 pretrain --arch llama --dims-json dims.json --model-name llama3_8B --total-flops 1e18 \\
        --data-dir /data/fineweb10B --out runs/llama_8B

(``--dims NAME`` is short for the packaged ``configs/model_dims.json``; ``--train-shards`` / ``--val-shards`` also take
a file path or glob directly.)  With dims given by flags, ``n_heads = d_model / head_dim``, ``n_kv_heads = n_heads``
and the FFN width ``8/3 * d_model`` rounded up to a multiple of ``head_dim`` are filled in when omitted.

The budget is ``--total-tokens`` (K / M / B suffixes) or ``--total-flops`` under ``6 * N * T`` accounting.  The output
directory receives ``meta.json`` (dims, hyper-parameters, derived totals), ``train.jsonl`` (every ``--log-every``
steps: step, loss, lr, tok/s, tokens seen, wall time), ``eval.jsonl`` (every ``--eval-every`` steps: val loss and
perplexity, eval time) and ``final.json``; a run whose ``final.json`` exists is skipped, which is the resume
convention of the scaling-law grid."""
from __future__ import annotations

import argparse
import glob
import json
import math
import os
import time
from typing import List, Optional

_SUFFIX = {"K": 10 ** 3, "M": 10 ** 6, "B": 10 ** 9, "T": 10 ** 12}


def parse_count(text) -> int:
    """``"1B"`` / ``"250M"`` / ``"16384"`` / ``"2.5e9"`` -> int."""
    if isinstance(text, (int, float)):
        return int(text)
    t = str(text).strip().upper().replace("_", "")
    if t and t[-1] in _SUFFIX:
        return int(float(t[:-1]) * _SUFFIX[t[-1]])
    return int(float(t))


def add_model_flags(p: argparse.ArgumentParser) -> None:
    p.add_argument("--arch", default=None, help="llama, mistral, qwen2, qwen3, qwen3_moe, olmoe, gemma2, gemma3, gemma4, "
                                                "qwen3_next, qwen3_5, qwen3_5_moe (default: the dims entry's, else llama)")
    p.add_argument("--dims", default=None, help="name in the packaged configs/model_dims.json, or a JSON file of one model")
    p.add_argument("--dims-json", default=None, help="JSON file keyed by model name")
    p.add_argument("--model-name", default=None, help="key into --dims-json")
    p.add_argument("--d-model", type=int)
    p.add_argument("--n-layers", type=int)
    p.add_argument("--vocab-size", type=int, default=None)
    p.add_argument("--n-heads", type=int)
    p.add_argument("--n-kv-heads", type=int)
    p.add_argument("--head-dim", type=int, default=None)
    p.add_argument("--expert-dim", type=int, help="FFN width (per expert for MoE)")
    p.add_argument("--num-routed-experts", type=int)
    p.add_argument("--top-k", type=int)
    p.add_argument("--shared-expert-dim", type=int, help="shared-expert FFN width (Qwen3-Next, Qwen3.5-MoE)")
    p.add_argument("--layer-pattern", help="hybrid schedule shorthand, e.g. 3L1F (F full, L linear, S sliding)")
    p.add_argument("--init-seed", "--seed", dest="init_seed", type=int, default=42)
    p.add_argument("--init-std", "--std", dest="init_std", type=float, default=0.02)
    p.add_argument("--max-seq-len", "--seq-len", dest="max_seq_len", type=int, default=1024)
    p.add_argument("--max-gpu-gib", "--max-gpu-mem-gib", dest="max_gpu_gib", type=float, default=None)
    p.add_argument("--max-host-gib", "--max-host-mem-gib", dest="max_host_gib", type=float, default=None)


def resolve_model(args):
    """``(arch, dims, hyperparams)`` from the model flags; raises ``SystemExit`` with a message on bad input."""
    hyper = None
    if args.dims_json:
        if not args.model_name:
            raise SystemExit("--dims-json also needs --model-name")
        with open(args.dims_json) as f:
            table = json.load(f)
        if args.model_name not in table:
            raise SystemExit(f"{args.model_name!r} is not in {args.dims_json} (has {sorted(table)[:8]}...)")
        dims = dict(table[args.model_name])
    elif args.dims:
        dims = dict(_load_dims(args.dims))
    else:
        if not args.d_model or not args.n_layers:
            raise SystemExit("need --d-model and --n-layers, or --dims / --dims-json + --model-name")
        hd = args.head_dim or 64
        if args.d_model % hd:
            raise SystemExit(f"--d-model ({args.d_model}) must be divisible by --head-dim ({hd})")
        n_heads = args.n_heads or args.d_model // hd
        ffn = args.expert_dim or -(-(8 * args.d_model // 3) // hd) * hd
        E = args.num_routed_experts or 0
        dims = dict(vocab_size=args.vocab_size or 50304, n_layers=args.n_layers, d_model=args.d_model, n_heads=n_heads,
                    n_kv_heads=args.n_kv_heads or n_heads, head_dim=hd, expert_dim=ffn, ffn_dim=ffn,
                    num_routed_experts=E, top_k=args.top_k or 0, num_shared_experts=0, is_causal=True)
        if args.shared_expert_dim:
            dims.update(num_shared_experts=1, shared_dim=args.shared_expert_dim)
    arch = args.arch or dims.pop("arch", None) or "llama"
    dims.pop("arch", None)
    hyper = dims.pop("hyperparams", None)
    if args.vocab_size and (args.dims or args.dims_json):
        dims["vocab_size"] = args.vocab_size
    if args.layer_pattern:
        hyper = {**(hyper or {}), "layer_pattern": args.layer_pattern}
    return arch, dims, hyper


def add_subparser(sub) -> None:
    p = sub.add_parser("pretrain", help="random-init pretraining on uint16 token shards",
                       formatter_class=argparse.RawDescriptionHelpFormatter, description=__doc__)
    add_model_flags(p)
    g = p.add_mutually_exclusive_group()
    g.add_argument("--total-tokens", "--token-budget", dest="total_tokens", default=None,
                   help="train for this many tokens (K / M / B suffixes)")
    g.add_argument("--total-flops", "--flop-budget", dest="total_flops", type=float, default=None,
                   help="train for this many FLOPs under 6 * N * T accounting")
    p.add_argument("--data-dir", default=None, help="directory with fineweb_train_NNNNNN.bin / fineweb_val_NNNNNN.bin")
    p.add_argument("--train-shards", default="1-99", help="range '1-99', list '1,2,3', or a path / glob")
    p.add_argument("--val-shard", "--val-shards", dest="val_shard", default=None,
                   help="val shard index (with --data-dir; default 0), or a path / glob")
    p.add_argument("--out", required=True, help="output directory")
    p.add_argument("--batch-tokens", type=int, default=16384)
    p.add_argument("--peak-lr", "--lr", dest="peak_lr", type=float, default=3.0e-4)
    p.add_argument("--warmup-frac", "--warmup-pct", dest="warmup_frac", type=float, default=0.02)
    p.add_argument("--weight-decay", type=float, default=0.1)
    p.add_argument("--grad-clip", type=float, default=None, help="clip the global gradient norm (off by default)")
    p.add_argument("--eval-every", type=int, default=200)
    p.add_argument("--eval-tokens", type=int, default=200_000)
    p.add_argument("--log-every", type=int, default=20)
    p.add_argument("--use-muon", action="store_true", help="Muon for the 2-D hidden weights, AdamW for the rest")
    p.add_argument("--device", default=None)
    p.set_defaults(func=run)


def _load_dims(name: str) -> dict:
    if os.path.exists(name):
        with open(name) as f:
            return json.load(f)
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(here, "configs", "model_dims.json")) as f:
        table = json.load(f)
    if name not in table:
        raise SystemExit(f"{name!r} is neither a file nor a packaged model (has {sorted(table)[:8]}...)")
    return table[name]


def resolve_shards(data_dir: Optional[str], spec: str, kind: str) -> List[str]:
    """``'1-99'`` / ``'1,2,5-7'`` with ``data_dir`` -> existing ``fineweb_<kind>_NNNNNN.bin`` paths; anything else is
    taken as a path or glob."""
    spec = str(spec)
    numeric = all(c.isdigit() or c in ",- " for c in spec) and any(c.isdigit() for c in spec)
    if data_dir and numeric:
        idx: List[int] = []
        for part in spec.split(","):
            part = part.strip()
            if "-" in part:
                a, b = part.split("-", 1)
                idx += list(range(int(a), int(b) + 1))
            elif part:
                idx.append(int(part))
        paths = [os.path.join(data_dir, f"fineweb_{kind}_{i:06d}.bin") for i in idx]
        found = [p for p in paths if os.path.exists(p)]
        if not found:
            raise FileNotFoundError(f"none of the {len(paths)} {kind} shards {spec!r} exist under {data_dir}")
        return found
    pat = os.path.join(data_dir, spec) if data_dir and not os.path.isabs(spec) and not os.path.exists(spec) else spec
    found = sorted(glob.glob(pat)) if any(c in pat for c in "*?[") else ([pat] if os.path.exists(pat) else [])
    if not found:
        raise FileNotFoundError(f"no shard matches {pat!r}")
    return found


def lr_at(step: int, steps: int, peak: float, warmup_frac: float, floor: float = 0.1) -> float:
    """Linear warm-up over ``warmup_frac`` of the run, then cosine decay to ``floor * peak`` (1-based ``step``)."""
    warm = max(1, int(steps * warmup_frac))
    if step <= warm:
        return peak * step / warm
    return peak * (floor + (1 - floor) * 0.5 * (1 + math.cos(math.pi * (step - warm) / max(1, steps - warm))))


def run(args) -> int:
    import torch

    import flextrain_b200 as ft
    from ..core._memory import get_available_gpu_memory, get_available_host_memory
    from ..core._sizing import model_param_count
    os.makedirs(args.out, exist_ok=True)
    final = os.path.join(args.out, "final.json")
    if os.path.exists(final):
        print(f"[pretrain] {final} exists; nothing to do")
        return 0
    arch, dims, hyper = resolve_model(args)
    device = args.device or ("cuda:0" if torch.cuda.is_available() else "cpu")
    cuda = device.startswith("cuda")
    n_params = model_param_count({"n_kv_heads": dims.get("n_heads"), **dims})
    flops_per_token = 6.0 * n_params
    if args.total_tokens is not None:
        budget_tokens = parse_count(args.total_tokens)
    elif args.total_flops is not None:
        budget_tokens = int(math.ceil(args.total_flops / flops_per_token))
    else:
        raise SystemExit("need --total-tokens or --total-flops")
    steps = max(1, -(-budget_tokens // args.batch_tokens))
    adamw = ft.AdamW(lr=args.peak_lr, weight_decay=args.weight_decay, state_dtype=torch.float32)
    opt = ft.HybridMuonAdamW(muon=ft.Muon(lr=args.peak_lr), adamw=adamw) if args.use_muon else adamw
    dt = torch.bfloat16 if cuda else torch.float32
    am = ft.from_dims(dims, arch=arch, hyperparams=hyper, optimizer=opt, max_seq_len=args.max_seq_len,
                      max_global_batch_tokens=args.batch_tokens,
                      max_gpu_mem_bytes=int(args.max_gpu_gib * 2 ** 30) if args.max_gpu_gib
                      else get_available_gpu_memory(device),
                      max_host_mem_bytes=int(args.max_host_gib * 2 ** 30) if args.max_host_gib
                      else get_available_host_memory(),
                      device=device, compute_dtype=dt, master_dtype=dt, grad_dtype=dt, init_on_device=cuda,
                      init_seed=args.init_seed, init_std=args.init_std)
    train_files = resolve_shards(args.data_dir, args.train_shards, "train")
    train = ft.ShardTokenSource(train_files, args.max_seq_len)
    val = None
    if args.val_shard is not None or args.data_dir:
        try:
            val = ft.ShardTokenSource(resolve_shards(args.data_dir, args.val_shard if args.val_shard is not None else "0",
                                                     "val"), args.max_seq_len, loop=True)
        except FileNotFoundError:
            if args.val_shard is not None:
                raise
    with open(os.path.join(args.out, "meta.json"), "w") as f:
        json.dump({"arch": arch, "dims": dims, "hyperparams": hyper, "n_params": n_params, "total_steps": steps,
                   "batch_tokens": args.batch_tokens, "total_tokens": budget_tokens, "total_flops": args.total_flops,
                   "peak_lr": args.peak_lr, "warmup_frac": args.warmup_frac, "weight_decay": args.weight_decay,
                   "max_seq_len": args.max_seq_len, "init_seed": args.init_seed, "init_std": args.init_std,
                   "optimizer": "muon+adamw" if args.use_muon else "adamw", "train_shards": train_files}, f, indent=1)
    t0, tokens, window = time.time(), 0, []
    last_t, last_tok, val_loss = t0, 0, None
    with open(os.path.join(args.out, "train.jsonl"), "a") as tl, open(os.path.join(args.out, "eval.jsonl"), "a") as el:
        for step in range(1, steps + 1):
            lr = lr_at(step, steps, args.peak_lr, args.warmup_frac)
            am.optimizer.lr = lr
            st = am.fwd_bwd(train.get_sequences(args.batch_tokens))
            am.step(max_grad_norm=args.grad_clip) if args.grad_clip else am.step()
            am.check_health()           # raises when a bounded device-side wait ran out during this step
            tokens += st.tokens
            window = (window + [st.loss])[-20:]
            if step % args.log_every == 0 or step == steps or step == 1:
                now = time.time()
                tl.write(json.dumps({"step": step, "loss": st.loss, "lr": lr,
                                     "tok_per_s": (tokens - last_tok) / max(now - last_t, 1e-9), "tokens_seen": tokens,
                                     "wall_time": now - t0}) + "\n")
                tl.flush()
                last_t, last_tok = now, tokens
            if val is not None and (step % args.eval_every == 0 or step == steps):
                te = time.time()
                val_loss = evaluate(am, val, args.eval_tokens, args.batch_tokens)
                el.write(json.dumps({"step": step, "val_loss": val_loss, "val_ppl": math.exp(min(val_loss, 50.0)),
                                     "eval_time_s": time.time() - te, "tokens_seen": tokens}) + "\n")
                el.flush()
    with open(final, "w") as f:
        json.dump({"steps": steps, "tokens": tokens, "seconds": time.time() - t0,
                   "train_loss": sum(window) / max(len(window), 1), "last_train_loss": window[-1] if window else None,
                   "val_loss": val_loss, "flops": flops_per_token * tokens, "n_params": n_params}, f, indent=1)
    return 0


def evaluate(am, source, eval_tokens: int, batch_tokens: int) -> float:
    """Mean loss over ``eval_tokens`` under the current weights (forward only; nothing of the training state moves)."""
    tot, n = 0.0, 0
    while n < eval_tokens:
        seqs = source.get_sequences(min(batch_tokens, eval_tokens - n) or batch_tokens)
        if not seqs:
            break
        st = am.evaluate(seqs)
        tot += st.loss_sum
        n += st.active_tokens
    return tot / max(n, 1)
