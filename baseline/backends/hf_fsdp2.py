"""Third-party baseline trainer: a HuggingFace ``transformers`` causal LM under PyTorch FSDP2 on synthetic tokens.

    python baseline/backends/hf_fsdp2.py --preset llama3_1_8B --seq-length 1024 --micro-batch-size 8 \
        --gradient-accumulation-steps 8 --num-steps 3
    python -m torch.distributed.run --nproc-per-node 8 ... baseline/backends/hf_fsdp2.py ...

The model is built from a config (random init) unless ``--model-path`` names an HF directory; it runs the stock HF
modelling code with autograd, ``torch.optim.AdamW(fused=True)`` and, for more than one rank,
``torch.distributed.fsdp.fully_shard`` per decoder layer.  Prints one ``step N: ... tok/s`` line per step in the format
``baseline/scripts/sweep.py`` extracts.  Nothing of flextrain_b200 is imported except the dims catalogue (a JSON).
"""
from __future__ import annotations

import argparse
import json
import os
import time

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def hf_config_from_preset(preset: str, n_layers=None):
    from transformers import LlamaConfig
    with open(os.path.join(ROOT, "flextrain_b200", "configs", "model_dims.json")) as f:
        cat = json.load(f)
    key = preset if preset in cat else next((k for k in cat if k.lower() == preset.lower()), None)
    if key is None:
        raise KeyError(f"unknown preset {preset!r}; known: {', '.join(sorted(cat))}")
    d = cat[key].get("dims", cat[key])
    return LlamaConfig(vocab_size=d["vocab_size"], hidden_size=d["d_model"],
                       intermediate_size=d.get("ffn_dim", d.get("expert_dim")),
                       num_hidden_layers=int(n_layers or d["n_layers"]), num_attention_heads=d["n_heads"],
                       num_key_value_heads=d["n_kv_heads"], head_dim=d["head_dim"], rms_norm_eps=1e-5,
                       rope_theta=500000.0, max_position_embeddings=131072, tie_word_embeddings=False)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="llama3_1_8B")
    ap.add_argument("--model-path", default=None)
    ap.add_argument("--seq-length", type=int, default=1024)
    ap.add_argument("--micro-batch-size", type=int, default=1)
    ap.add_argument("--gradient-accumulation-steps", type=int, default=1)
    ap.add_argument("--num-steps", type=int, default=3)
    ap.add_argument("--warmup-steps", type=int, default=1)
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--n-layers", type=int, default=None)
    ap.add_argument("--activation-checkpointing", action="store_true")
    ap.add_argument("--cpu-offload", action="store_true")
    ap.add_argument("--attn-implementation", default="sdpa")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    from transformers import AutoModelForCausalLM

    rank, world, local = (int(os.environ.get(k, d)) for k, d in (("RANK", 0), ("WORLD_SIZE", 1), ("LOCAL_RANK", 0)))
    torch.cuda.set_device(local)
    dev = torch.device(f"cuda:{local}")
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.manual_seed(args.seed)
    if args.model_path:
        model = AutoModelForCausalLM.from_pretrained(args.model_path, torch_dtype=torch.bfloat16,
                                                     attn_implementation=args.attn_implementation)
    else:
        cfg = hf_config_from_preset(args.preset, args.n_layers)
        cfg._attn_implementation = args.attn_implementation
        with torch.device("meta"):
            model = AutoModelForCausalLM.from_config(cfg, torch_dtype=torch.bfloat16)
        model.to_empty(device=dev)
        for p in model.parameters():
            torch.nn.init.normal_(p, 0.0, 0.02) if p.dim() > 1 else torch.nn.init.ones_(p)
    model.to(dev)
    if args.activation_checkpointing:
        model.gradient_checkpointing_enable()
    model.config.use_cache = False
    if world > 1:
        from torch.distributed.fsdp import CPUOffloadPolicy, fully_shard
        kw = {"offload_policy": CPUOffloadPolicy()} if args.cpu_offload else {}
        for layer in model.model.layers:
            fully_shard(layer, **kw)
        fully_shard(model, **kw)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-5, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0, fused=True)
    vocab = model.config.vocab_size
    gen = torch.Generator().manual_seed(args.seed + rank)
    tokens_per_step = args.seq_length * args.micro_batch_size * args.gradient_accumulation_steps * world
    model.train()
    for step in range(args.warmup_steps + args.num_steps):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        loss_sum = 0.0
        for _ in range(args.gradient_accumulation_steps):
            ids = torch.randint(0, vocab, (args.micro_batch_size, args.seq_length), generator=gen).pin_memory()
            ids = ids.to(dev, non_blocking=True)
            out = model(input_ids=ids, labels=ids)
            (out.loss / args.gradient_accumulation_steps).backward()
            loss_sum += float(out.loss.detach())
        opt.step()
        opt.zero_grad(set_to_none=True)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t)
        if rank == 0:
            tag = "warmup" if step < args.warmup_steps else "step"
            print(f"{tag} {step}: loss {loss_sum / args.gradient_accumulation_steps:.4f}  {dt * 1e3:.1f} ms  "
                  f"{tokens_per_step / dt:.1f} tok/s  max_alloc {torch.cuda.max_memory_allocated() / 2**30:.1f} GiB",
                  flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
