"""Random-init a model from a dims spec and export it as an HF directory (``config.json`` + ``model.safetensors``)
(flextrain/scripts/init_hf.py:1-30).  The model is named like in ``pretrain``: ``--dims NAME``, ``--dims-json FILE
--model-name KEY``, or ``--d-model / --n-layers / ...`` flags."""
from __future__ import annotations


def add_subparser(sub) -> None:
    from .pretrain import add_model_flags
    p = sub.add_parser("init", help="write a randomly initialised HF model directory from a dims spec")
    add_model_flags(p)
    p.add_argument("--out", required=True)
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.set_defaults(func=run, init_seed=0xF1EC7)


def run(args) -> int:
    import torch

    import flextrain_b200 as ft
    from ..engine.host_memory import UnpinnedHostBackend
    from ..export import save_hf_full
    from .pretrain import resolve_model
    arch, dims, hyper = resolve_model(args)
    dt = getattr(torch, args.dtype)
    am = ft.from_dims(dims, arch=arch, hyperparams=hyper, optimizer=ft.AdamW(), max_seq_len=128,
                      max_global_batch_tokens=128, max_gpu_mem_bytes=1 << 40, max_host_mem_bytes=1 << 40, device="cpu",
                      compute_dtype=dt, master_dtype=dt, grad_dtype=dt, init_seed=args.init_seed, init_std=args.init_std,
                      working_set=ft.WorkingSetConfig.simple(max_seq_len=128, max_global_batch_tokens=128),
                      host_backend=UnpinnedHostBackend())
    save_hf_full(am, args.out)
    print(f"[init] wrote {args.out} ({arch}, {sum(t.numel() for _, _, _, t in am.named_master_params()):,} parameters)")
    return 0
