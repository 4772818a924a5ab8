"""Worker for the engine-level expert- and tensor-parallel tests (run under ``torch.distributed.run``).

``ep``: every rank builds the same small Qwen3-MoE model with ``ep = world`` (experts sharded over the ranks, the rest
data parallel) and trains on its share of the batch.  ``tp``: a small Llama with ``tp = world`` (heads and FFN width
sharded, token-sharded residual stream); every rank feeds the whole batch.  After a few steps the parameters are
gathered back through the HF exporter; rank 0 also trains the unsharded model on the whole batch in the same process
and reports the differences.  ``tp_ragged``: as ``tp`` with sequences of uneven lengths (one of them longer than a
chunk), so chunk token counts are not multiples of the shard width and the scheduler has to pad them.
``ep_ragged``: as ``ep`` with uneven sequences split unevenly over the ranks, so the ranks' chunks differ in length
and one rank has more rounds and more chunks than the other (it is padded with filler chunks).
``tp_hostopt``: as ``tp`` with the optimizer state kept in host memory and streamed through a two-slot device ring
during ``step()`` (what a 70B model over 8 tensor-parallel ranks needs); results must equal the resident run.
``ep_lora``: as ``ep`` with LoRA on every projection, including per-expert adapters on the sharded expert stacks; the
merged weights (base + adapters, gathered) must match the unsharded run.
``ep_clip``: as ``ep`` with global gradient-norm clipping (the norm sums the expert parts over the group).
``ep_muon``: as ``ep`` with the hybrid optimizer: Muon orthogonalises each expert matrix of the local stack and the
replicated hidden matrices (after their gradients were reduced), AdamW takes the rest.
``tp_grid`` / ``ep_grid``: model-parallel groups of two ranks inside a larger job (a ``dp x tp`` / ``dp x ep`` grid over
library collectives); every group trains on its share of the batch.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import flextrain_b200 as ft  # noqa: E402
from flextrain_b200.io.hf_weights import collect_hf_state  # noqa: E402

MOE_DIMS = dict(vocab_size=512, n_layers=2, d_model=128, n_heads=4, n_kv_heads=2, head_dim=32, expert_dim=64,
                ffn_dim=64, num_routed_experts=8, num_shared_experts=0, top_k=2, is_causal=True)
DENSE_DIMS = dict(vocab_size=512, n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, expert_dim=512,
                  ffn_dim=512, num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)
GB, SEQ, STEPS = 1024, 128, 2
RAGGED = [100, 37, 300, 77, 41, 131, 65, 29, 200]      # 980 tokens; the 300-token one spans two 256-token chunks


def build(dev, dtype, world, rank, mode, backend):
    from flextrain_b200.engine.host_memory import UnpinnedHostBackend
    os.environ["FTB_DP_BACKEND"] = backend
    mp = 2 if mode.endswith("_grid") else world                # model-parallel group size
    per_rank = GB // max(world // mp, 1) if mode.startswith("tp") else GB // world
    ragged = mode in ("tp_ragged", "ep_ragged")
    seq = 512 if ragged else SEQ
    ws = ft.WorkingSetConfig.simple(max_seq_len=seq, max_global_batch_tokens=per_rank,
                                    chunk=256 if ragged else 512,
                                    round_tokens=512 if mode == "ep_ragged" else per_rank, world_size=world,
                                    shard="opt+grad" if world > 1 else "none",
                                    **({"n_gpu_opt_layers": 2} if mode == "tp_hostopt" and world > 1 else {}))
    par = {"ep": mp} if mode.startswith("ep") else {"tp": mp}
    lora = dict(lora_targets="all", lora_rank=4, lora_alpha=8.0, lora_adapter_compute_dtype=dtype,
                lora_adapter_master_dtype=dtype, lora_adapter_grad_dtype=dtype,
                lora_adapter_opt_state_dtype=torch.float32) if mode in ("tp_lora", "ep_lora") else {}
    hybrid = mode == "ep_hybrid"        # Gated DeltaNet + gated attention layers, routed + shared experts
    gemma = mode == "tp_gemma"          # sandwich norms, per-head QK-norm, sliding + global layers, tied scaled embedding
    hyper = {"sliding_window": 64, "layer_pattern": "SF"} if gemma else None
    dims = MOE_DIMS if mode.startswith("ep") else DENSE_DIMS
    if hybrid:
        dims = dict(MOE_DIMS, num_shared_experts=1, shared_dim=64)
        hyper = {"layer_pattern": "1L1F", "gdn": {"n_k_heads": 2, "n_v_heads": 4, "head_k_dim": 16, "head_v_dim": 16}}
    return ft.from_dims(dims,
                        arch="qwen3_5_moe" if hybrid else "qwen3_moe" if mode.startswith("ep") else ("gemma3" if gemma else "llama"),
                        hyperparams=hyper,
                        optimizer=(ft.HybridMuonAdamW(muon=ft.Muon(lr=1e-3, state_dtype=torch.float32),
                                                      adamw=ft.AdamW(lr=1e-3, state_dtype=torch.float32))
                                   if mode == "ep_muon" else ft.AdamW(lr=1e-3, state_dtype=torch.float32)),
                        max_seq_len=seq, max_global_batch_tokens=GB, max_gpu_mem_bytes=8 << 30,
                        max_host_mem_bytes=8 << 30, device=dev, compute_dtype=dtype, master_dtype=dtype,
                        grad_dtype=dtype, working_set=ws, world_size=world, rank=rank,
                        host_backend=UnpinnedHostBackend() if dev == "cpu" else None, **lora,
                        **(par if world > 1 else {}))


def train(am, rank, world, dev, mode):
    ragged = mode in ("tp_ragged", "ep_ragged")
    src = ft.SyntheticTokenSource(512, RAGGED if ragged else SEQ, seed=5)
    losses = []
    for _ in range(4 if mode in ("tp_lora", "ep_lora") else STEPS):      # LoRA: B starts at zero, A only moves from step 2 on
        seqs = src.get_sequences(sum(RAGGED) if ragged else GB)
        if mode.startswith("ep"):
            seqs = seqs[rank::world]                  # data parallel: each rank takes its share of the batch
        elif mode == "tp_grid" and world > 1:
            seqs = seqs[rank // 2::world // 2]        # each tensor-parallel pair takes its share
        st = am.fwd_bwd(seqs, loss_scale_factor=1.0 / GB, total_tokens_per_step=GB)
        assert am.step(max_grad_norm=0.05 if mode == "ep_clip" else None) == 0      # 0.05: every step clips
        t = torch.tensor([st.loss_sum], device=dev, dtype=torch.float64 if dev == "cpu" else torch.float32)
        if world > 1:
            dist.all_reduce(t)
        losses.append(float(t) / GB)
    return losses


def main():
    backend, mode, out_path = sys.argv[1], sys.argv[2], sys.argv[3]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    if backend == "p2p":
        torch.cuda.set_device(local)
        dev, dtype = f"cuda:{local}", torch.bfloat16
        dist.init_process_group("nccl", device_id=torch.device(dev))
    else:
        dev, dtype = "cpu", torch.float32
        dist.init_process_group("gloo")
    am = build(dev, dtype, world, rank, mode, backend)
    local_rows = am.buffers.params(0)["w_up" if mode.startswith("ep") else "w_1"].shape[0]
    if mode == "tp_ragged" and world > 1:
        from flextrain_b200.engine.schedule import prepare_training_chunks
        probe = ft.SyntheticTokenSource(512, RAGGED, seed=5).get_sequences(sum(RAGGED))
        metas = prepare_training_chunks(probe, 256, dev, pad_multiple=128 * world)
        assert all(m.num_tokens % (128 * world) == 0 for m in metas) and sum(m.extra["pad_tokens"] for m in metas) > 0
    losses = train(am, rank, world, dev, mode)
    if am.ep is not None:
        am.ep.check()
    merge = mode in ("tp_lora", "ep_lora")        # compare base + adapters, merged: the adapters are what trained
    state = collect_hf_state(am, lora_merge=merge)      # collective: gathers the tensor- / expert-parallel parts
    adapters = {}
    if mode in ("tp_lora", "ep_lora"):            # gather every adapter (collective) for a direct comparison
        from flextrain_b200.io.hf_weights import gather_local_parts
        for l, layer in enumerate(am.layers):
            for n, t in am.buffers.host_params(l).items():
                if "_lora_" in n:
                    spec = layer.param_spec.get(n)
                    adapters[(l, n)] = (gather_local_parts(t.detach(), spec, am) if spec.is_local_part else t.detach()).float().cpu()
    adapter_dir = out_path + ".adapter"
    if mode in ("tp_lora", "ep_lora"):
        from flextrain_b200.export import save_lora_adapter
        save_lora_adapter(am, adapter_dir)        # collective gather of the sharded adapters; rank 0 writes
    res = None
    if rank == 0:
        full = build(dev, dtype, 1, 0, mode, backend)
        ref_losses = train(full, 0, 1, dev, mode)
        ref_state = collect_hf_state(full, lora_merge=merge)
        worst = 0.0
        for k, v in ref_state.items():
            d = float((state[k].float() - v.float()).abs().max())
            worst = max(worst, d)
        res = {"local_rows": int(local_rows), "loss_diff": max(abs(a - b) for a, b in zip(losses, ref_losses)),
               "param_diff": worst, "losses": losses, "keys": len(ref_state)}
        if adapters:
            worst_a, moved = 0.0, 0.0
            for l in range(len(full.layers)):
                for n, t in full.buffers.host_params(l).items():
                    if "_lora_" in n:
                        worst_a = max(worst_a, float((adapters[(l, n)] - t.detach().float().cpu()).abs().max()))
                        if n.endswith("_lora_b"):
                            moved = max(moved, float(t.detach().abs().max()))
            res["adapter_diff"], res["adapter_moved"] = worst_a, moved
            from safetensors import safe_open
            with safe_open(os.path.join(adapter_dir, "adapter_model.safetensors"), framework="pt") as f:
                res["adapter_file_shapes"] = {k: list(f.get_tensor(k).shape) for k in f.keys() if "layers.0." in k}
        if backend == "p2p":
            from flextrain_b200.ops import cuda as k
            res["errors"] = k.device_error_words()
        with open(out_path, "w") as f:
            json.dump(res, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
