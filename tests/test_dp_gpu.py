"""Peer-memory data parallelism on 2+ B200s: fused reduce-scatter + sharded AdamW with parameter push, checked
against the library-collective baseline (NCCL all-reduce + replicated AdamW)."""
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(backend, out, n):
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "dp_worker.py"), backend, out]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return torch.load(out)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_p2p_matches_collective(tmp_path):
    n = min(torch.cuda.device_count(), 4)
    a = _run("p2p", str(tmp_path / "p2p.pt"), n)
    b = _run("collective", str(tmp_path / "coll.pt"), n)
    assert a["ranks_identical"] and b["ranks_identical"]
    assert "comm" in a["libs"], "peer-memory kernels were not loaded"
    assert all(v == 0 for v in a["errors"].values()), a["errors"]
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 2e-2, (a["losses"], b["losses"])
    d = (a["params"] - b["params"]).abs()
    # the sharded path keeps fp32 reduced gradients, the baseline rounds the all-reduce to bf16: tiny drift only
    assert float(d.mean()) < 2e-4 and float(d.max()) < 2e-2, (float(d.mean()), float(d.max()))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_deferred_param_gather_fused_into_qkv_gemm(tmp_path):
    """``opt+grad+param``: the optimizer writes only its own range and the next step's QKV projection of each layer
    pulls the rest of the layer out of peer memory inside the GEMM kernel; results match the eager-push path."""
    n = min(torch.cuda.device_count(), 4)
    a = _run("p2p_param", str(tmp_path / "p2pp.pt"), n)
    b = _run("p2p", str(tmp_path / "p2p.pt"), n)
    assert a["deferred_layers"] == [0, 1, 2], a["deferred_layers"]
    assert a["ranks_identical"]
    assert all(v == 0 for v in a["errors"].values()), a["errors"]
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 1e-3, (a["losses"], b["losses"])
    d = (a["params"] - b["params"]).abs()
    # the gather-GEMM runs on the one-SM kernel, the eager path's projection on the two-SM kernel: a different fp32
    # summation order, i.e. single-ulp bf16 differences after three updates
    assert float(d.mean()) < 1e-5 and float(d.max()) < 5e-3, (float(d.mean()), float(d.max()))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_fwd_bwd_calls_per_step_match_one_call(tmp_path):
    """Gradient accumulation over two ``fwd_bwd`` calls before ``step()``: each call takes its own flag epoch, so the
    second reduce-scatter waits for the peers' second backward; parameters match the one-call run of the same batch."""
    n = min(torch.cuda.device_count(), 4)
    a = _run("p2p_accum", str(tmp_path / "acc.pt"), n)
    b = _run("p2p", str(tmp_path / "one.pt"), n)
    assert a["ranks_identical"] and all(v == 0 for v in a["errors"].values()), a["errors"]
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 2e-3, (a["losses"], b["losses"])
    d = (a["params"] - b["params"]).abs()
    assert float(d.mean()) < 2e-5 and float(d.max()) < 5e-3, (float(d.mean()), float(d.max()))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_gradient_clipping_on_shards_matches_collective(tmp_path):
    """``step(max_grad_norm=...)`` on the peer-memory path takes the norm from the reduced fp32 shards (one scalar
    all-reduce) and scales the shard; the library-collective path clips whole replicated gradients."""
    n = min(torch.cuda.device_count(), 4)
    a = _run("p2p_clip", str(tmp_path / "p2p.pt"), n)
    b = _run("collective_clip", str(tmp_path / "coll.pt"), n)
    assert a["ranks_identical"] and all(v == 0 for v in a["errors"].values()), a["errors"]
    assert len(a["norms"]) == 3 and all(x > 0.05 for x in a["norms"]), a["norms"]
    for x, y in zip(a["norms"], b["norms"]):
        assert abs(x - y) < 0.02 * y, (a["norms"], b["norms"])
    d = (a["params"] - b["params"]).abs()
    assert float(d.mean()) < 2e-4 and float(d.max()) < 2e-2, (float(d.mean()), float(d.max()))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_hybrid_muon_on_peer_memory_path_matches_collective(tmp_path):
    """Muon tensors are reduced to one owner rank each, updated there (Newton-Schulz on the tcgen05 GEMM) and pushed
    to the peers by stores; AdamW tensors stay sharded by element range.  Against NCCL all-reduce + replicated step."""
    n = min(torch.cuda.device_count(), 4)
    a = _run("p2p_muon", str(tmp_path / "p2p.pt"), n)
    b = _run("collective_muon", str(tmp_path / "coll.pt"), n)
    assert a["ranks_identical"] and all(v == 0 for v in a["errors"].values()), a["errors"]
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 3e-2, (a["losses"], b["losses"])
    d = (a["params"] - b["params"]).abs()
    # Newton-Schulz in bf16 amplifies the bf16-vs-fp32 difference of the reduced gradient a little
    assert float(d.mean()) < 5e-4 and float(d.max()) < 5e-2, (float(d.mean()), float(d.max()))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_in_switch_gradient_reduction_matches_peer_loads(tmp_path):
    """``FTB_DP_MULTIMEM=1``: the gradient arena is bound to an NVSwitch multicast object and every rank pulls the sum of
    its range with ``multimem.ld_reduce`` (added inside the switch) instead of loading each peer's copy.  bf16 sums are
    rounded once by the switch, so parameters agree with the peer-load path to bf16 round-off."""
    n = min(torch.cuda.device_count(), 4)
    a = _run("p2p_mm", str(tmp_path / "mm.pt"), n)
    if not a["multicast"]:
        pytest.skip("this platform reports no NVLink multicast support")
    b = _run("p2p", str(tmp_path / "p2p.pt"), n)
    assert a["ranks_identical"] and all(v == 0 for v in a["errors"].values()), a["errors"]
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 2e-2, (a["losses"], b["losses"])
    d = (a["params"] - b["params"]).abs()
    assert float(d.mean()) < 2e-4 and float(d.max()) < 2e-2, (float(d.mean()), float(d.max()))
