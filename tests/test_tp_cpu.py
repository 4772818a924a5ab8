"""Tensor parallelism in the engine on CPU (gloo, 2 ranks, library collectives): heads and FFN width sharded, the
residual stream token-sharded; losses and re-gathered parameters match the unsharded single-process run."""
import json
import os
import socket
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def test_engine_tensor_parallel_matches_unsharded(tmp_path):
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "tpe.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "parallel_engine_worker.py"), "collective", "tp",
           out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert res["local_rows"] == 256            # w_1 holds ffn_dim / 2 rows on each rank
    assert res["loss_diff"] < 1e-4 and res["param_diff"] < 1e-3, res


def test_engine_tensor_parallel_pads_ragged_chunks(tmp_path):
    """Sequences of uneven lengths (one longer than a chunk): chunk token counts are rounded up to the shard multiple
    with unscored filler after the last real token; losses, per-token write-back and the trained parameters still
    match the unsharded, unpadded run."""
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "tpr.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "parallel_engine_worker.py"), "collective",
           "tp_ragged", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert res["loss_diff"] < 1e-4 and res["param_diff"] < 1e-3, res


def test_engine_tensor_parallel_gemma_layer_shape(tmp_path):
    """Sandwich (pre + post) norms on the token-sharded branch outputs, per-head QK-norm whose replicated gains see
    different heads per rank, sliding and global layers, tied scaled embedding: two ranks match the unsharded run."""
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "tpg.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "parallel_engine_worker.py"), "collective",
           "tp_gemma", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert res["loss_diff"] < 1e-4 and res["param_diff"] < 1e-3, res


def test_engine_tensor_parallel_lora(tmp_path):
    """LoRA on sharded weights: the adapter on a weight's sharded side is sharded with it, the other one is replicated
    and its partial gradients are summed by the data-parallel reduction; four steps (both adapters move) match the
    unsharded LoRA run, compared through the merged weights."""
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "tpl.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "parallel_engine_worker.py"), "collective",
           "tp_lora", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert res["loss_diff"] < 1e-4 and res["param_diff"] < 1e-4, res
    assert res["adapter_moved"] > 1e-3 and res["adapter_diff"] < 1e-2 * res["adapter_moved"], res
    shapes = res["adapter_file_shapes"]                        # the PEFT file holds whole adapters, not shards
    assert shapes["base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight"] == [256, 4]
    assert shapes["base_model.model.model.layers.0.self_attn.o_proj.lora_A.weight"] == [4, 256]
    assert shapes["base_model.model.model.layers.0.mlp.down_proj.lora_A.weight"] == [4, 512]


def test_engine_grid_of_tensor_parallel_pairs(tmp_path):
    """Four ranks as a 2 x 2 grid (two tensor-parallel pairs, data parallel across the pairs) over library collectives:
    replicated tensors are reduced over the job, each pair's parts over their replicas; losses and the re-gathered
    parameters match the single-process run on the whole batch."""
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "grid.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "parallel_engine_worker.py"), "collective",
           "tp_grid", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert res["local_rows"] == 256 and res["loss_diff"] < 1e-4 and res["param_diff"] < 1e-3, res


def test_tensor_spec_localisation():
    import torch
    from flextrain_b200.core.layer import TensorSpec
    t = TensorSpec("w_up", (8, 6, 4), torch.float32).localize(0, 1, 4)
    assert t.shape == (2, 6, 4) and t.global_shape == (8, 6, 4) and t.local_slice == (0, 2, 4) and t.is_local_part
    u = TensorSpec("w_o", (16, 4), torch.float32).mark_local(1, 2, 4)
    assert u.shape == (16, 4) and u.global_shape == (16, 16) and u.local_slice == (1, 8, 12)
    assert not TensorSpec("w_attn_norm", (16,), torch.float32).is_local_part


def test_muon_is_refused_under_tensor_parallelism():
    import pytest
    import torch
    import flextrain_b200 as ft
    dims = dict(vocab_size=512, n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, expert_dim=512,
                ffn_dim=512, num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)
    with pytest.raises(NotImplementedError, match="Muon"):
        ft.from_dims(dims, optimizer=ft.HybridMuonAdamW(), max_seq_len=128, max_global_batch_tokens=512,
                     max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30, device="cpu", world_size=2, rank=0, tp=2,
                     plan_only=True)


def test_engine_tensor_parallel_with_host_resident_optimizer_state(tmp_path):
    """Tensor parallelism with the optimizer state in host memory, streamed through a two-slot ring in ``step()``
    (the layout the planner picks for a 70B model on 8 GPUs): two ranks match the unsharded, fully resident run."""
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "tph.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "parallel_engine_worker.py"), "collective",
           "tp_hostopt", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert res["loss_diff"] < 1e-4 and res["param_diff"] < 1e-3, res
