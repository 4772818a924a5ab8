"""Book-keeping helpers: FLOP accounting of a step, parameter counts, batch-size divisors, memory probes and the YAML
run configuration."""
import pytest
import torch

import flextrain_b200 as ft
from flextrain_b200.config import RunConfig
from flextrain_b200.core import flop_accounting as fa
from flextrain_b200.core.memory import get_available_gpu_memory, get_available_host_memory
from flextrain_b200.core.sizing import divisors, layer_param_count, matmul_flops_per_token, model_param_count, prev_high_div
from conftest import build_tiny

DIMS = dict(vocab_size=256, n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, expert_dim=128, ffn_dim=128,
            num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)


def test_step_flops_follow_the_6n_rule_plus_attention():
    am = build_tiny(dims=DIMS, max_seq_len=64, batch_tokens=128)
    seqs = ft.SyntheticTokenSource(256, 64, seed=0).get_sequences(128)
    st = am.fwd_bwd(seqs)
    n_layer = sum(t.numel() for s, l, n, t in am.named_master_params() if s == "layer" and t.dim() == 2)
    attn = st.attn_fwd_flops
    assert st.fwd_flops == pytest.approx(2.0 * n_layer * 128 + attn, rel=1e-6)       # 2 FLOPs per weight per token
    eff, hw = fa.step_flops_breakdown(am, st, mode="full")
    head = fa.head_flops(am, 128)
    assert head == 2.0 * 128 * 256 * 64
    assert eff == pytest.approx(3.0 * st.fwd_flops + 3.0 * head + fa.opt_flops_per_step(am), rel=1e-9)
    assert hw >= eff                                                                # hardware FLOPs add recompute / rescan
    lora_eff, _ = fa.step_flops_breakdown(am, st, mode="lora")
    assert lora_eff < eff                                                           # no weight gradients of the base
    n_train = sum(t.numel() for _, _, _, t in am.named_master_params())
    assert fa.opt_flops_per_step(am) == 12.0 * n_train
    am.optimizer = ft.HybridMuonAdamW()
    assert fa.opt_flops_per_step(am) > 12.0 * n_train and fa.opt_ns_iters(am.optimizer) == 5


def test_parameter_counts_and_divisors():
    d = dict(DIMS)
    attn = 64 * 64 + 2 * 64 * 32 + 64 * 64
    assert layer_param_count(d) == attn + 3 * 64 * 128 + 2 * 64
    assert model_param_count(d) == 2 * layer_param_count(d) + 2 * 256 * 64 + 64
    assert matmul_flops_per_token(d) == pytest.approx(2.0 * (2 * (attn + 3 * 64 * 128) + 256 * 64))
    moe = dict(d, expert_dim=32, num_routed_experts=8, top_k=2)
    assert matmul_flops_per_token(moe, active_only=True) < matmul_flops_per_token(moe, active_only=False)
    assert divisors(36) == [1, 2, 3, 4, 6, 9, 12, 18, 36]
    v = prev_high_div(524288 + 777)
    assert v <= 524288 + 777 and v % 1024 == 0 and len(divisors(v // 1024)) >= 10
    assert prev_high_div(500) == 500


def test_memory_probes():
    host = get_available_host_memory()
    assert isinstance(host, int) and host > (64 << 20)
    assert get_available_gpu_memory("cpu") == 8 << 30          # the CPU engine's nominal "device" budget
    assert get_available_gpu_memory("cuda:0") >= 0             # 0 when no GPU answers, never an exception


def test_run_config_from_yaml(tmp_path):
    p = tmp_path / "c.yaml"
    p.write_text("model: {dims: tiny_llama, mode: lora, lora_rank: 4}\noptimizer: {name: muon, lr: 2.0e-3}\n"
                 "train: {steps: 7, max_seq_len: 64, max_global_batch_tokens: 256}\nhardware: {tp: 2}\n"
                 "data: {source: synthetic}\nio: {output_dir: out, save_state_every: 3}\nunknown_section: {x: 1}\n")
    c = RunConfig.from_yaml(str(p))
    assert (c.model.dims, c.model.mode, c.model.lora_rank) == ("tiny_llama", "lora", 4)
    assert c.optimizer.name == "muon" and c.optimizer.lr == 2e-3 and c.train.steps == 7 and c.hardware.tp == 2
    assert c.io.save_state_every == 3 and c.io.resume_state is None
    from flextrain_b200.cli import _train_argv
    argv = _train_argv(c)
    assert "--use-muon" in argv and argv[argv.index("--tp") + 1] == "2" and argv[argv.index("--save-state-every") + 1] == "3"
    assert RunConfig.from_dict({}).train.steps > 0                                  # defaults fill everything


def test_reference_style_optimizer_constructors_and_package_exports():
    """``AdamW(AdamWHyperparams(...), state_dtype=...)`` / ``Muon(MuonHyperparams(...))`` build the same optimizers as
    the keyword form, and the sub-packages export the names a user of the reference imports from them."""
    import torch
    from flextrain_b200.optim import AdamW, AdamWHyperparams, Muon, MuonHyperparams, state_key
    a = AdamW(AdamWHyperparams(lr=3e-5, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.0), state_dtype=torch.float32)
    assert a == AdamW(lr=3e-5, weight_decay=0.0, state_dtype=torch.float32) and a.hp.lr == 3e-5
    assert Muon(MuonHyperparams(lr=2e-3, ns_iters=3)).ns_iters == 3
    assert state_key("o_adam_m", "w_q") == "o_adam_m_q"
    from flextrain_b200.engine import (BufferManager, ChunkPolicy, EventBook, LocalPinnedHostBackend, StreamBundle,  # noqa: F401
                                        default_host_backend, prepare_training_chunks, split_sequences,
                                        unregister_all_process_pinned_memory)
    from flextrain_b200.core import (ActivationSchema, ChunkMeta, HardwareCost, Layer, ParamSpec, SaveLevelPlan,  # noqa: F401
                                      TensorSpec, build_dp_tables, probe_hardware)
    from flextrain_b200.nn import IGNORE_INDEX, CrossEntropyLoss, LMHead, TokenEmbedLayer  # noqa: F401
    from flextrain_b200.io import Sequence, ShardTokenSource, SyntheticTokenSource, TokenSource  # noqa: F401
    assert IGNORE_INDEX == -100 and unregister_all_process_pinned_memory() == 0
