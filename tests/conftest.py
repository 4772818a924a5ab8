import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "multigpu: needs 2 or more CUDA devices")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords or "multigpu" in item.keywords:
            item.add_marker(skip)


TINY_DIMS = dict(vocab_size=1024, n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, expert_dim=688,
                 ffn_dim=688, num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)


@pytest.fixture
def tiny_dims():
    return dict(TINY_DIMS)


def build_tiny(arch="llama", dims=None, hyper=None, optimizer=None, ws=None, device="cpu", dtype=torch.float32,
               max_seq_len=128, batch_tokens=256, **kw):
    import flextrain_b200 as ft
    from flextrain_b200.engine.host_memory import UnpinnedHostBackend
    dims = dict(dims or TINY_DIMS)
    optimizer = optimizer or ft.AdamW(lr=1e-3, state_dtype=torch.float32, beta2=0.95)
    ws = ws or ft.WorkingSetConfig.simple(max_seq_len=max_seq_len, max_global_batch_tokens=batch_tokens)
    return ft.from_dims(dims, arch=arch, optimizer=optimizer, max_seq_len=max_seq_len,
                        max_global_batch_tokens=batch_tokens, max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30,
                        hyperparams=hyper, device=device, compute_dtype=dtype, master_dtype=dtype, grad_dtype=dtype,
                        working_set=ws, host_backend=UnpinnedHostBackend() if device == "cpu" else None, **kw)
