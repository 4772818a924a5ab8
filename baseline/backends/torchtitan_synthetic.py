"""Third-party baseline trainer: TorchTitan's Llama-3 model, FSDP2 sharding and activation checkpointing on synthetic tokens.

    python baseline/backends/torchtitan_synthetic.py --preset llama3_1_8B --seq-length 1024 --micro-batch-size 8 \
        --gradient-accumulation-steps 8 --num-steps 3 --ac-mode full
    python -m torch.distributed.run --nproc-per-node 8 ... baseline/backends/torchtitan_synthetic.py ...

Everything on the training path is TorchTitan's or PyTorch's: ``torchtitan.models.llama3.Transformer`` built from
``TransformerModelArgs`` (dims from this repository's catalogue JSON), its ``init_weights``, its cross-entropy loss,
``apply_ac`` / ``apply_fsdp`` from ``torchtitan.models.llama3.infra.parallelize`` (per-block ``fully_shard`` with bf16
parameters and fp32 reduction), ``torch.optim.AdamW(fused=True)``.  Random token ids stand in for a text dataset, as in
the reference project's TorchTitan registry (baseline/backends/torchtitan/synthetic_registry.py there).  Prints one
``step N: ... tok/s`` line per step in the format ``baseline/scripts/sweep.py`` extracts.  Nothing of flextrain_b200 is
imported.
"""
from __future__ import annotations

import argparse
import json
import os
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def model_args_from_preset(preset: str, seq_len: int, n_layers=None):
    """``TransformerModelArgs`` whose derived FFN width equals the catalogue's (TorchTitan derives it from
    ``ffn_dim_multiplier`` and ``multiple_of``: hidden = multiple_of * ceil(multiplier * (8 d / 3) / multiple_of))."""
    from torchtitan.models.llama3 import TransformerModelArgs
    with open(os.path.join(ROOT, "flextrain_b200", "configs", "model_dims.json")) as f:
        cat = json.load(f)
    key = preset if preset in cat else next((k for k in cat if k.lower() == preset.lower()), None)
    if key is None:
        raise KeyError(f"unknown preset {preset!r}; known: {', '.join(sorted(cat))}")
    d = cat[key].get("dims", cat[key])
    dim, ffn = int(d["d_model"]), int(d.get("ffn_dim", d.get("expert_dim")))
    if d["head_dim"] * d["n_heads"] != dim:
        raise ValueError("TorchTitan's Llama ties head_dim to dim / n_heads; this preset does not")
    base = int(2 * (4 * dim) / 3)
    multiple = next(m for m in (1024, 512, 256, 128, 64, 32, 16, 8, 1) if ffn % m == 0)
    mult = ffn / base
    args = TransformerModelArgs(dim=dim, n_layers=int(n_layers or d["n_layers"]), n_heads=int(d["n_heads"]),
                                n_kv_heads=int(d["n_kv_heads"]), vocab_size=int(d["vocab_size"]), multiple_of=multiple,
                                ffn_dim_multiplier=mult, norm_eps=1e-5, rope_theta=500000.0, max_seq_len=seq_len)
    got = multiple * ((int(mult * base) + multiple - 1) // multiple)
    if got != ffn:                       # float rounding in the multiplier: nudge it until the derived width matches
        for eps in (1e-9, -1e-9, 1e-7, -1e-7, 1e-5, -1e-5):
            if multiple * ((int((mult + eps) * base) + multiple - 1) // multiple) == ffn:
                args.ffn_dim_multiplier = mult + eps
                break
        else:
            raise ValueError(f"cannot express FFN width {ffn} for dim {dim} through TorchTitan's multiplier")
    return args


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="llama3_1_8B")
    ap.add_argument("--seq-length", type=int, default=1024)
    ap.add_argument("--micro-batch-size", type=int, default=1)
    ap.add_argument("--gradient-accumulation-steps", type=int, default=1)
    ap.add_argument("--num-steps", type=int, default=3)
    ap.add_argument("--warmup-steps", type=int, default=1)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--n-layers", type=int, default=None)
    ap.add_argument("--ac-mode", choices=("none", "selective", "full"), default="full")
    ap.add_argument("--cpu-offload", action="store_true")
    ap.add_argument("--device", default=None, help="cpu runs a smoke pass of the same code without FSDP")
    args = ap.parse_args(argv)

    import torch
    import torch.distributed as dist
    from torchtitan.components.loss import cross_entropy_loss as loss_fn
    from torchtitan.models.llama3 import Transformer

    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    cuda = (args.device or "cuda").startswith("cuda") and torch.cuda.is_available()
    dev = torch.device(f"cuda:{local}" if cuda else "cpu")
    if cuda:
        torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": dev} if cuda else {}))
    torch.manual_seed(args.seed)
    margs = model_args_from_preset(args.preset, args.seq_length, args.n_layers)
    with torch.device("meta"):
        model = Transformer(margs)
    if args.ac_mode != "none":
        from torchtitan.config.job_config import ActivationCheckpoint
        from torchtitan.models.llama3.infra.parallelize import apply_ac
        apply_ac(model, ActivationCheckpoint(mode=args.ac_mode, selective_ac_option="op"))
    if world > 1:
        from torch.distributed.device_mesh import init_device_mesh
        from torchtitan.models.llama3.infra.parallelize import apply_fsdp
        mesh = init_device_mesh(dev.type, (world,), mesh_dim_names=("dp_shard",))
        apply_fsdp(model, mesh, param_dtype=torch.bfloat16, reduce_dtype=torch.float32, pp_enabled=False,
                   cpu_offload=args.cpu_offload)
    model.to_empty(device=dev)
    with torch.no_grad():
        model.init_weights(buffer_device=dev)
    if world == 1 and cuda:
        model.to(torch.bfloat16)                          # one GPU: plain bf16 parameters (FSDP's mixed precision is off)
    model.train()
    opt = torch.optim.AdamW(model.parameters(), lr=3e-5, betas=(0.9, 0.95), weight_decay=0.0, fused=cuda)
    n_params = sum(p.numel() for p in model.parameters()) * (world if world > 1 else 1)
    mb, ga, S, V = args.micro_batch_size, args.gradient_accumulation_steps, args.seq_length, margs.vocab_size
    g = torch.Generator(device="cpu").manual_seed(args.seed + rank)
    tokens_per_step = mb * ga * S * world
    for step in range(1, args.warmup_steps + args.num_steps + 1):
        if cuda:
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        total = 0.0
        for _ in range(ga):
            ids = torch.randint(0, V, (mb, S + 1), generator=g)
            ids = ids.pin_memory().to(dev, non_blocking=True) if cuda else ids
            logits = model(ids[:, :-1])
            loss = loss_fn(logits, ids[:, 1:]) / ga
            loss.backward()
            total += float(loss.detach())
        opt.step()
        opt.zero_grad(set_to_none=True)
        if cuda:
            torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if rank == 0:
            tag = "warmup " if step <= args.warmup_steps else ""
            mem = torch.cuda.max_memory_allocated() / 2 ** 30 if cuda else 0.0
            print(f"{tag}step {step}: loss {total:.4f} step_time {dt:.3f}s tok/s {tokens_per_step / dt:,.0f} "
                  f"max_alloc {mem:.1f}GiB params {n_params / 1e9:.2f}B", flush=True)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
