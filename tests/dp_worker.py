"""Worker run under ``torch.distributed.run`` by test_dp_gpu.py: trains a small Llama for a few steps with the
chosen data-parallel backend and writes rank 0's parameters and losses to a file."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import flextrain_b200 as ft  # noqa: E402


def main():
    backend, out_path = sys.argv[1], sys.argv[2]
    shard = "opt+grad"
    accum = backend.endswith("_accum")      # the step's batch in two fwd_bwd calls (gradient accumulation over calls)
    backend = backend.replace("_accum", "")
    clip = 0.05 if backend.endswith("_clip") else None       # well below the norm of these gradients: every step clips
    backend = backend.replace("_clip", "")
    if backend.endswith("_mm"):             # gradient reduce-scatter as in-switch reductions (multimem.ld_reduce)
        os.environ["FTB_DP_MULTIMEM"] = "1"
        backend = backend[:-3]
    hybrid = backend.endswith("_muon")      # Muon for the hidden matrices, AdamW for the rest
    backend = backend.replace("_muon", "")
    if backend == "p2p_param":              # peer-memory path with the parameter all-gather deferred into the QKV GEMM
        backend, shard = "p2p", "opt+grad+param"
    os.environ["FTB_DP_BACKEND"] = backend
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    dims = dict(vocab_size=2048, n_layers=3, d_model=512, n_heads=4, n_kv_heads=2, head_dim=128, expert_dim=1408,
                num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)
    gb = 4096
    adamw = ft.AdamW(lr=1e-3, state_dtype=torch.float32, weight_decay=0.01)
    am = ft.from_dims(dims, arch="llama",
                      optimizer=ft.HybridMuonAdamW(muon=ft.Muon(lr=2e-3), adamw=adamw) if hybrid else adamw,
                      max_seq_len=256, max_global_batch_tokens=gb, max_gpu_mem_bytes=16 << 30,
                      max_host_mem_bytes=16 << 30, device=dev, world_size=world, rank=rank,
                      working_set=ft.WorkingSetConfig.simple(max_seq_len=256, max_global_batch_tokens=gb // world,
                                                             chunk=1024, round_tokens=1024, world_size=world,
                                                             shard=shard))
    src = ft.SyntheticTokenSource(2048, 256, seed=11)
    losses, norms = [], []
    for step in range(3):
        seqs = src.get_sequences(gb)[rank::world]
        if accum:
            h = len(seqs) // 2
            st = am.fwd_bwd(seqs[:h], loss_scale_factor=1.0 / gb, total_tokens_per_step=gb)
            st2 = am.fwd_bwd(seqs[h:], loss_scale_factor=1.0 / gb, total_tokens_per_step=gb)
            st.loss_sum += st2.loss_sum
        else:
            st = am.fwd_bwd(seqs, loss_scale_factor=1.0 / gb, total_tokens_per_step=gb)
        assert am.step(max_grad_norm=clip) == 0
        if clip is not None:
            norms.append(am.last_grad_norm)
        t = torch.tensor([st.loss_sum], device=dev)
        dist.all_reduce(t)
        losses.append(float(t) / gb)
    if hasattr(am.dp, "finish_param_gather"):
        deferred = sorted(am.dp._stale)
        am.dp.finish_param_gather()
    else:
        deferred = []
    torch.cuda.synchronize()
    if hasattr(am.dp, "check"):
        am.dp.check()
    flat = torch.cat([t.flatten().float().cpu() for _, _, _, t in am.named_master_params()])
    allflat = [None] * world
    dist.all_gather_object(allflat, flat)
    if rank == 0:
        same = all(torch.equal(allflat[0], f) for f in allflat)
        from flextrain_b200.ops import cuda as k
        torch.save({"params": flat, "losses": losses, "ranks_identical": same, "errors": k.device_error_words(),
                    "libs": sorted(k._libs), "deferred_layers": deferred, "norms": norms,
                    "multicast": bool(getattr(getattr(am.buffers, "grad_arena", None), "mc_ptr", 0))}, out_path)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
