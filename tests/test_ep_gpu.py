"""Expert-parallel dispatch / combine over peer memory on 2+ GPUs against the single-GPU MoE block."""
import json
import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_p2p(tmp_path):
    n = 2 if torch.cuda.device_count() < 4 else 4
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "ep.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "ep_worker.py"), "p2p", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert all(v == 0 for v in res.pop("errors").values())
    for k, v in res.items():
        assert v < 3e-2, (k, v, res)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_engine_expert_parallel_p2p(tmp_path):
    """A small Qwen3-MoE trained with experts sharded over 2 GPUs (peer-memory dispatch / combine, sharded AdamW for
    the replicated part, local AdamW for the experts) against the unsharded model on one GPU."""
    s = socket.socket(); s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]; s.close()
    out = str(tmp_path / "epe.json")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "parallel_engine_worker.py"), "p2p", "ep", out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = json.load(open(out))
    assert all(v == 0 for v in res.pop("errors").values())
    assert res["local_rows"] == 4
    assert res["loss_diff"] < 2e-2 and res["param_diff"] < 2e-2, res
