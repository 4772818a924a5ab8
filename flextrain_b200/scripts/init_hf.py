"""Random-init a dims spec and export it as an HF directory (``config.json`` + ``model.safetensors``)
(flextrain/scripts/init_hf.py:1-30)."""
from __future__ import annotations

import json
import os


def add_subparser(sub) -> None:
    p = sub.add_parser("init", help="write a randomly initialised HF model directory from a dims spec")
    p.add_argument("--dims", required=True)
    p.add_argument("--out", required=True)
    p.add_argument("--seed", type=int, default=0xF1EC7)
    p.add_argument("--std", type=float, default=0.02)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.set_defaults(func=run)


def run(args) -> int:
    import torch

    import flextrain_b200 as ft
    from ..engine.host_memory import UnpinnedHostBackend
    from ..export import save_hf_full
    from .pretrain import _load_dims
    dims = dict(_load_dims(args.dims))
    arch, hyper = dims.pop("arch", "llama"), dims.pop("hyperparams", None)
    dt = getattr(torch, args.dtype)
    am = ft.from_dims(dims, arch=arch, hyperparams=hyper, optimizer=ft.AdamW(), max_seq_len=128,
                      max_global_batch_tokens=128, max_gpu_mem_bytes=1 << 40, max_host_mem_bytes=1 << 40, device="cpu",
                      compute_dtype=dt, master_dtype=dt, grad_dtype=dt, init_seed=args.seed, init_std=args.std,
                      working_set=ft.WorkingSetConfig.simple(max_seq_len=128, max_global_batch_tokens=128),
                      host_backend=UnpinnedHostBackend())
    save_hf_full(am, args.out)
    print(f"[init] wrote {args.out}")
    return 0
