"""Worker for the engine-level expert-parallel tests (run under ``torch.distributed.run``).

Every rank builds the same small Qwen3-MoE model with ``ep = world``: experts are sharded over the ranks, the rest is
data parallel.  Trains a few steps on its share of the batch, then gathers the parameters back through the HF
exporter; rank 0 also trains the unsharded model on the whole batch in the same process and reports the differences.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import flextrain_b200 as ft  # noqa: E402
from flextrain_b200.io.hf_weights import collect_hf_state  # noqa: E402

DIMS = dict(vocab_size=512, n_layers=2, d_model=128, n_heads=4, n_kv_heads=2, head_dim=32, expert_dim=64, ffn_dim=64,
            num_routed_experts=8, num_shared_experts=0, top_k=2, is_causal=True)
GB, SEQ, STEPS = 1024, 128, 2


def build(dev, dtype, world, rank, ep, backend):
    from flextrain_b200.engine.host_memory import UnpinnedHostBackend
    os.environ["FTB_DP_BACKEND"] = backend
    ws = ft.WorkingSetConfig.simple(max_seq_len=SEQ, max_global_batch_tokens=GB // world, chunk=256,
                                    round_tokens=GB // world, world_size=world,
                                    shard="opt+grad" if world > 1 else "none")
    return ft.from_dims(DIMS, arch="qwen3_moe", optimizer=ft.AdamW(lr=1e-3, state_dtype=torch.float32),
                        max_seq_len=SEQ, max_global_batch_tokens=GB, max_gpu_mem_bytes=8 << 30,
                        max_host_mem_bytes=8 << 30, device=dev, compute_dtype=dtype, master_dtype=dtype,
                        grad_dtype=dtype, working_set=ws, world_size=world, rank=rank, ep=ep,
                        host_backend=UnpinnedHostBackend() if dev == "cpu" else None)


def train(am, rank, world, dev):
    src = ft.SyntheticTokenSource(DIMS["vocab_size"], SEQ, seed=5)
    losses = []
    for _ in range(STEPS):
        seqs = src.get_sequences(GB)[rank::world]
        st = am.fwd_bwd(seqs, loss_scale_factor=1.0 / GB, total_tokens_per_step=GB)
        assert am.step() == 0
        t = torch.tensor([st.loss_sum], device=dev, dtype=torch.float64 if dev == "cpu" else torch.float32)
        if world > 1:
            dist.all_reduce(t)
        losses.append(float(t) / GB)
    return losses


def main():
    backend, out_path = sys.argv[1], sys.argv[2]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    if backend == "p2p":
        torch.cuda.set_device(local)
        dev, dtype = f"cuda:{local}", torch.bfloat16
        dist.init_process_group("nccl", device_id=torch.device(dev))
    else:
        dev, dtype = "cpu", torch.float32
        dist.init_process_group("gloo")
    am = build(dev, dtype, world, rank, world, backend)
    local_experts = am.buffers.params(0)["w_up"].shape[0]
    losses = train(am, rank, world, dev)
    if am.ep is not None:
        am.ep.check()
    state = collect_hf_state(am)                  # collective: gathers the expert shards
    res = None
    if rank == 0:
        full = build(dev, dtype, 1, 0, 1, backend)
        ref_losses = train(full, 0, 1, dev)
        ref_state = collect_hf_state(full)
        worst = 0.0
        for k, v in ref_state.items():
            d = float((state[k].float() - v.float()).abs().max())
            worst = max(worst, d)
        res = {"local_experts": int(local_experts), "loss_diff": max(abs(a - b) for a, b in zip(losses, ref_losses)),
               "param_diff": worst, "losses": losses, "keys": len(ref_state)}
        if backend == "p2p":
            from flextrain_b200.ops import cuda as k
            res["errors"] = k.device_error_words()
        with open(out_path, "w") as f:
            json.dump(res, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
