"""Random-init pretraining on token shards with token / FLOP budgets and periodic evaluation
(flextrain/scripts/pretrain.py:1-44, 518-571).  Writes ``meta.json``, ``train.jsonl``, ``eval.jsonl`` and
``final.json``; a run whose ``final.json`` exists is skipped."""
from __future__ import annotations

import argparse
import json
import os
import time


def add_subparser(sub) -> None:
    p = sub.add_parser("pretrain", help="random-init pretraining on uint16 token shards")
    p.add_argument("--dims", required=True, help="name in configs/model_dims.json or a JSON file")
    p.add_argument("--train-shards", required=True)
    p.add_argument("--val-shards", default=None)
    p.add_argument("--out", required=True)
    p.add_argument("--seq-len", type=int, default=1024)
    p.add_argument("--batch-tokens", type=int, default=131072)
    p.add_argument("--token-budget", type=int, default=None)
    p.add_argument("--flop-budget", type=float, default=None)
    p.add_argument("--lr", type=float, default=6e-4)
    p.add_argument("--warmup-pct", type=float, default=0.02)
    p.add_argument("--eval-every", type=int, default=100)
    p.add_argument("--eval-tokens", type=int, default=262144)
    p.add_argument("--use-muon", action="store_true")
    p.add_argument("--max-gpu-mem-gib", type=float, default=None)
    p.add_argument("--device", default=None)
    p.set_defaults(func=run)


def _load_dims(name: str) -> dict:
    if os.path.exists(name):
        with open(name) as f:
            return json.load(f)
    here = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(here, "configs", "model_dims.json")) as f:
        return json.load(f)[name]


def run(args) -> int:
    import math

    import torch

    import flextrain_b200 as ft
    from ..core.memory import get_available_gpu_memory, get_available_host_memory
    from ..core.sizing import model_param_count
    os.makedirs(args.out, exist_ok=True)
    final = os.path.join(args.out, "final.json")
    if os.path.exists(final):
        print(f"[pretrain] {final} exists; nothing to do")
        return 0
    dims = dict(_load_dims(args.dims))
    arch, hyper = dims.pop("arch", "llama"), dims.pop("hyperparams", None)
    device = args.device or ("cuda:0" if torch.cuda.is_available() else "cpu")
    cuda = device.startswith("cuda")
    n_params = model_param_count({"n_kv_heads": dims.get("n_heads"), **dims})
    flops_per_token = 6.0 * n_params
    budget_tokens = args.token_budget or int((args.flop_budget or 1e15) / flops_per_token)
    steps = max(1, budget_tokens // args.batch_tokens)
    opt = ft.HybridMuonAdamW(muon=ft.Muon(lr=args.lr), adamw=ft.AdamW(lr=args.lr, state_dtype=torch.float32)) \
        if args.use_muon else ft.AdamW(lr=args.lr, weight_decay=0.1, state_dtype=torch.float32)
    dt = torch.bfloat16 if cuda else torch.float32
    am = ft.from_dims(dims, arch=arch, hyperparams=hyper, optimizer=opt, max_seq_len=args.seq_len,
                      max_global_batch_tokens=args.batch_tokens,
                      max_gpu_mem_bytes=int(args.max_gpu_mem_gib * 2 ** 30) if args.max_gpu_mem_gib
                      else get_available_gpu_memory(device), max_host_mem_bytes=get_available_host_memory(),
                      device=device, compute_dtype=dt, master_dtype=dt, grad_dtype=dt, init_on_device=cuda)
    train = ft.ShardTokenSource(args.train_shards, args.seq_len)
    val = ft.ShardTokenSource(args.val_shards, args.seq_len, loop=True) if args.val_shards else None
    with open(os.path.join(args.out, "meta.json"), "w") as f:
        json.dump({"dims": dims, "arch": arch, "n_params": n_params, "steps": steps, "batch_tokens": args.batch_tokens,
                   "token_budget": budget_tokens, "lr": args.lr}, f, indent=1)
    warm = max(1, int(steps * args.warmup_pct))
    t0, tokens = time.time(), 0
    tl, el = open(os.path.join(args.out, "train.jsonl"), "a"), open(os.path.join(args.out, "eval.jsonl"), "a")
    val_loss = None
    for step in range(1, steps + 1):
        am.optimizer.lr = args.lr * step / warm if step <= warm else \
            args.lr * (0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * (step - warm) / max(1, steps - warm))))
        seqs = train.get_sequences(args.batch_tokens)
        st = am.fwd_bwd(seqs)
        am.step()
        tokens += st.tokens
        tl.write(json.dumps({"step": step, "loss": st.loss, "tokens": tokens, "elapsed": time.time() - t0}) + "\n")
        tl.flush()
        if val is not None and (step % args.eval_every == 0 or step == steps):
            val_loss = evaluate(am, val, args.eval_tokens, args.batch_tokens)
            el.write(json.dumps({"step": step, "val_loss": val_loss, "tokens": tokens}) + "\n")
            el.flush()
    with open(final, "w") as f:
        json.dump({"steps": steps, "tokens": tokens, "seconds": time.time() - t0, "train_loss": st.loss,
                   "val_loss": val_loss, "flops": flops_per_token * tokens}, f, indent=1)
    return 0


def evaluate(am, source, eval_tokens: int, batch_tokens: int) -> float:
    """Mean loss over ``eval_tokens`` without touching the weights: forward+backward is run and the gradients
    are discarded (the engine's head computes the loss inside its fused forward/backward)."""
    tot, n = 0.0, 0
    while n < eval_tokens:
        seqs = source.get_sequences(min(batch_tokens, eval_tokens - n) or batch_tokens)
        if not seqs:
            break
        st = am.fwd_bwd(seqs)
        am._zero_grad = True
        tot += st.loss_sum
        n += st.active_tokens
    return tot / max(n, 1)
