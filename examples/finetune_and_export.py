"""API example: LoRA fine-tune a model, then write the three export formats
(flextrain examples/finetune_and_export.py).

    python examples/finetune_and_export.py --model <hf dir> [--steps 10]
    python examples/finetune_and_export.py --dims tiny_llama            # random-init toy model, runs on CPU
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import flextrain_b200 as ft  # noqa: E402
from flextrain_b200.export import save_hf_full, save_hf_merged, save_lora_adapter  # noqa: E402

if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default=None)
    ap.add_argument("--dims", default="tiny_llama")
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--out", default="runs/example_export")
    a = ap.parse_args()
    cuda = torch.cuda.is_available()
    dev, dt = ("cuda:0", torch.bfloat16) if cuda else ("cpu", torch.float32)
    common = dict(optimizer=ft.AdamW(lr=1e-4, state_dtype=torch.float32), max_seq_len=256, max_global_batch_tokens=2048,
                  max_gpu_mem_bytes=(torch.cuda.mem_get_info()[0] if cuda else 8 << 30), max_host_mem_bytes=32 << 30,
                  device=dev, compute_dtype=dt, master_dtype=dt, grad_dtype=dt, lora_targets="all", lora_rank=16,
                  lora_alpha=16.0, lora_adapter_compute_dtype=dt, lora_adapter_master_dtype=dt,
                  lora_adapter_grad_dtype=dt, lora_adapter_opt_state_dtype=torch.float32)
    if a.model:
        am = ft.from_pretrained(a.model, **common)
        vocab = am.model_config.vocab_size
    else:
        cat = json.load(open(os.path.join(os.path.dirname(ft.__file__), "configs", "model_dims.json")))
        dims = dict(cat[a.dims]); arch = dims.pop("arch"); hyper = dims.pop("hyperparams", None)
        am = ft.from_dims(dims, arch=arch, hyperparams=hyper, **common)
        vocab = dims["vocab_size"]
    src = ft.SyntheticTokenSource(vocab, 256, seed=0, pin=cuda)
    for step in range(a.steps):
        st = am.fwd_bwd(src.get_sequences(2048))
        am.step()
        print(f"step {step} loss {st.loss:.4f}")
    save_lora_adapter(am, os.path.join(a.out, "adapter"))
    save_hf_merged(am, os.path.join(a.out, "merged"))
    save_hf_full(am, os.path.join(a.out, "base_only"))
    print("exports written under", a.out)
