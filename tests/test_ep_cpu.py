"""Expert-parallel host logic on CPU (gloo, 2 ranks): the dispatch plan, combine and backward against the
single-process MoE block."""
import json
import os
import socket
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def test_expert_parallel_two_ranks_gloo(tmp_path):
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "ep.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "ep_worker.py"), "collective", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    for k, v in res.items():
        assert v < 1e-4, (k, v, res)


def test_engine_expert_parallel_matches_unsharded(tmp_path):
    """Two gloo ranks train a small Qwen3-MoE with the experts sharded (ep=2); losses and the re-gathered
    parameters match the unsharded single-process run on the same batch."""
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "epe.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "parallel_engine_worker.py"), "collective", "ep", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert res["local_rows"] == 4
    assert res["loss_diff"] < 1e-4 and res["param_diff"] < 1e-3, res


def test_engine_grid_of_expert_parallel_pairs(tmp_path):
    """Four gloo ranks as two expert-parallel pairs (each pair holds all experts once): tokens are dispatched inside a
    pair, expert gradients are reduced between the pairs' replicas, everything else over the job."""
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "epgrid.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=4", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "parallel_engine_worker.py"), "collective",
           "ep_grid", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert res["local_rows"] == 4
    assert res["loss_diff"] < 1e-4 and res["param_diff"] < 1e-3, res


def test_engine_expert_parallel_hybrid_with_shared_expert(tmp_path):
    """Qwen3.5-MoE layer shapes under ep=2: Gated DeltaNet and gated-attention mixers stay data parallel, routed experts
    are sharded, the sigmoid-gated shared expert is replicated; matches the unsharded run."""
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "eph.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "parallel_engine_worker.py"), "collective",
           "ep_hybrid", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert res["local_rows"] == 4 and res["loss_diff"] < 1e-4 and res["param_diff"] < 1e-3, res


def test_engine_expert_parallel_with_unequal_chunks_and_rounds(tmp_path):
    """Data-parallel ranks read different sequences: here rank 0 gets 706 tokens in 2 rounds / 4 + 1 chunks and rank 1
    274 tokens in 1 round / 2 chunks, with chunk lengths that differ between the ranks.  The symmetric buffers are sized
    from the planner's chunk size and the short rank runs filler chunks, so every dispatch / combine has its partner;
    losses and parameters match the unsharded single-process run on the whole batch."""
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "epr.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "parallel_engine_worker.py"), "collective",
           "ep_ragged", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert res["local_rows"] == 4 and res["loss_diff"] < 1e-4 and res["param_diff"] < 1e-3, res


def test_engine_expert_parallel_lora_with_per_expert_adapters(tmp_path):
    """ep=2 with LoRA on every projection: each rank holds the adapters of its own experts (3-D ``A`` / ``B`` sliced like
    the expert stacks), the dense adapters are replicated and reduced; the merged weights, gathered over the ranks, match
    the unsharded run."""
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "epl.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "parallel_engine_worker.py"), "collective",
           "ep_lora", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert res["local_rows"] == 4
    assert res["loss_diff"] < 1e-4 and res["param_diff"] < 1e-3, res
    # every adapter (gathered over the ranks) equals the unsharded run's, the adapters did move, and the PEFT file
    # written by rank 0 holds all 8 experts of layer 0 (4 of them live on the other rank)
    assert res["adapter_diff"] < 1e-3 and res["adapter_moved"] > 0, res
    shapes = res["adapter_file_shapes"]
    experts = {k.split(".experts.")[1].split(".")[0] for k in shapes if ".experts." in k}
    assert experts == {str(e) for e in range(8)}, sorted(experts)
    assert shapes["base_model.model.model.layers.0.mlp.experts.7.gate_proj.lora_A.weight"] == [4, 128]
    assert shapes["base_model.model.model.layers.0.mlp.experts.7.down_proj.lora_B.weight"] == [128, 4]


def test_engine_expert_parallel_with_hybrid_muon(tmp_path):
    """ep=2 with Muon on the hidden matrices: a rank orthogonalises the expert matrices it owns (a stack is a batch of
    matrices), replicated matrices are orthogonalised identically on both ranks after the gradient reduction; matches
    the unsharded run."""
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "epm.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "parallel_engine_worker.py"), "collective",
           "ep_muon", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert res["loss_diff"] < 1e-4 and res["param_diff"] < 2e-3, res


def test_engine_expert_parallel_gradient_clipping(tmp_path):
    """Global-norm clipping under ep=2: replicated tensors count once, the ranks' expert slices are summed over the
    group, so both ranks scale by the same factor as the unsharded run."""
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "epc.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "parallel_engine_worker.py"), "collective",
           "ep_clip", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert res["loss_diff"] < 1e-4 and res["param_diff"] < 1e-3, res
