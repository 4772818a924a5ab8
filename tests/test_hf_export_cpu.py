"""The other direction of the HuggingFace parity check: a model built and exported by the engine (``save_hf_full``)
must load in ``transformers`` with no missing tensor and give the engine's loss on the same tokens.  This pins the
exported ``config.json`` and the export side of every family's name map to the upstream definition
(the reference's analogue: tests/io/test_export_roundtrip_loss.py, which reloads into the reference itself)."""
import pytest
import torch

import flextrain_b200 as ft
from flextrain_b200.export import save_hf_full
from conftest import build_tiny
from test_arch_parity_cpu import CASES

transformers = pytest.importorskip("transformers")


@pytest.mark.parametrize("case", sorted(CASES))
def test_export_loads_in_transformers(case, tmp_path):
    arch, dims, hyper = CASES[case]
    am = build_tiny(arch=arch, dims=dims, hyper=hyper, max_seq_len=64, batch_tokens=128)
    torch.manual_seed(1)
    for _, _, name, t in am.named_master_params():
        if "norm" in name or "scalar" in name or name.startswith("b_"):
            t.add_(torch.randn_like(t) * 0.1)
    out = str(tmp_path / case)
    save_hf_full(am, out)
    model, info = transformers.AutoModelForCausalLM.from_pretrained(out, dtype=torch.float32,
                                                                    attn_implementation="eager",
                                                                    output_loading_info=True)
    assert not info["missing_keys"], info["missing_keys"]
    assert not info["unexpected_keys"], info["unexpected_keys"]
    seqs = ft.SyntheticTokenSource(dims["vocab_size"], 64, seed=0).get_sequences(128)
    st = am.fwd_bwd(seqs, loss_scale_factor=1.0)
    total = 0.0
    with torch.no_grad():
        for s in seqs:
            logits = model(input_ids=s.tokens[None].long()).logits[0].float()
            total += float(torch.nn.functional.cross_entropy(logits, s.targets.long(), ignore_index=-100,
                                                             reduction="sum"))
    assert abs(st.loss_sum - total) / total < 2e-4, (case, st.loss_sum, total)
