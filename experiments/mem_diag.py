"""Per-substep GPU memory trace used to calibrate the planner's workspace formula
(flextrain experiments/_mem_diag*.py): wraps the engine's forward / head / backward / step phases with
``torch.cuda.max_memory_allocated`` snapshots and prints the peak of each against the planner's estimate.

    python experiments/mem_diag.py --dims llama3_2_1B --seq-len 2048 --batch 65536
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import flextrain_b200 as ft  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--dims", default="llama3_2_1B")
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=65536)
    a = ap.parse_args()
    assert torch.cuda.is_available(), "needs a GPU"
    cat = json.load(open(os.path.join(os.path.dirname(ft.__file__), "configs", "model_dims.json")))
    dims = dict(cat[a.dims]); arch = dims.pop("arch"); hyper = dims.pop("hyperparams", None)
    free = torch.cuda.mem_get_info()[0]
    am = ft.from_dims(dims, arch=arch, hyperparams=hyper, optimizer=ft.AdamW(state_dtype=torch.float32),
                      max_seq_len=a.seq_len, max_global_batch_tokens=a.batch, max_gpu_mem_bytes=free,
                      max_host_mem_bytes=64 << 30, device="cuda:0", init_on_device=True, verbose=True)
    base = torch.cuda.memory_allocated()
    phases = {}
    for name in ("_forward_pass", "_backward_pass", "_step_local"):
        orig = getattr(am, name)

        def wrapped(*args, _o=orig, _n=name, **kw):
            torch.cuda.reset_peak_memory_stats()
            r = _o(*args, **kw)
            phases[_n] = max(phases.get(_n, 0), torch.cuda.max_memory_allocated())
            return r
        setattr(am, name, wrapped)
    src = ft.SyntheticTokenSource(dims["vocab_size"], a.seq_len, pin=True)
    am.fwd_bwd(src.get_sequences(a.batch)); am.step()
    print(f"resident state: {base / 2**30:.2f} GiB; planner activation room: {am.ws.gpu_act_buffer_size / 2**30:.2f} GiB")
    for k, v in phases.items():
        print(f"{k:16s} peak {v / 2**30:.2f} GiB (+{(v - base) / 2**30:.2f} over resident state)")
