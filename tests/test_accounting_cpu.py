"""Book-keeping helpers: FLOP accounting of a step, parameter counts, batch-size divisors, memory probes and the YAML
run configuration."""
import json
import os
import pytest
import torch

import flextrain_b200 as ft
from flextrain_b200.config import RunConfig
from flextrain_b200.core import flop_accounting as fa
from flextrain_b200.core._memory import get_available_gpu_memory, get_available_host_memory
from flextrain_b200.core._sizing import divisors, layer_param_count, matmul_flops_per_token, model_param_count, prev_high_div
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
                 "data: {source: synthetic}\nio: {output_dir: out, save_state_every: 3}\n")
    c = RunConfig.from_yaml(str(p))
    assert (c.model.dims, c.model.mode, c.model.lora_rank) == ("tiny_llama", "lora", 4)
    assert c.optimizer.name == "muon" and c.optimizer.lr == 2e-3 and c.train.steps == 7 and c.hardware.tp == 2
    assert c.io.save_state_every == 3 and c.io.resume_state is None
    from flextrain_b200.cli import _train_argv
    argv = _train_argv(c)
    assert "--use-muon" in argv and argv[argv.index("--tp") + 1] == "2" and argv[argv.index("--save-state-every") + 1] == "3"
    assert RunConfig.from_dict({}).train.steps > 0                                  # defaults fill everything
    for bad in ({"unknown_section": {"x": 1}}, {"train": {"stepz": 3}}):            # a typo is refused, not ignored
        with pytest.raises(ValueError, match="not understood"):
            RunConfig.from_dict(bad)


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


def test_engine_surface_answers_to_the_reference_spellings(tmp_path):
    """A training loop written against the reference runs unchanged: ``fwd_bwd(sequences=...)``, ``StepStats``'s
    ``total_loss / total_tokens / rounds``, ``step(step_num)``, ``save_hf(out_filename=...)``, ``load_hf(hf_path=...)``,
    ``am.working_set / backbone / step_count``, ``probe_hardware(...).hw_cost`` and ``register_block_builder`` with a
    list of architecture names."""
    import os
    import pytest
    import torch
    import flextrain_b200 as ft
    from conftest import build_tiny
    from flextrain_b200.core.hw_probe import probe_hardware
    am = build_tiny(batch_tokens=512)
    src = ft.SyntheticTokenSource(vocab_size=1024, seq_lens=128, seed=0)
    seqs = src.get_sequences(512)
    st = am.fwd_bwd(sequences=seqs, loss_scale_factor=1.0 / 512, total_tokens_per_step=512, verbose=False)
    assert st.total_tokens == 512 and st.rounds == st.n_rounds >= 1 and st.total_loss == st.loss_sum > 0
    assert am.step(7) == 0 and am.step_count == 7 and am.step() == 0 and am.step_count == 8
    assert am.working_set is am.ws and am.backbone is am.layers and am.hw_cost is am.hw
    assert am.dims["vocab_size"] == 1024 and am.dims["n_layers"] == len(am.backbone) and am.dims["expert_dim"] > 0
    with pytest.raises(TypeError):
        am.fwd_bwd()
    path = am.save_hf(str(tmp_path), out_filename="weights.safetensors")
    assert os.path.basename(path) == "weights.safetensors" and os.path.exists(path)
    before = am.evaluate(seqs).total_loss
    for _, _, _, t in am.named_master_params():
        t.zero_()
    am.load_hf(hf_path=str(tmp_path), strict=False)
    assert abs(am.evaluate(seqs).total_loss - before) < 1e-3 * before
    probe = probe_hardware(device="cpu", matmul_target_seconds=0.1, n_matmul_warmup=1)
    assert isinstance(probe, ft.HardwareCost) and probe.hw_cost.peak_tflops == probe.peak_tflops and probe.mem_bw_gbps > 0
    hw = ft.HardwareCost(peak_tflops=100.0, pcie_bw_gbps=10.0, practical_efficiency_factor=0.5)
    assert hw.flops_to_ms(1e14) == 2000.0 and hw.pcie_bytes_per_ms == 1e7 and hw.effective_flops_per_ms == 5e10
    plan = ft.SaveLevelPlan.uniform(2, 3, 1)
    assert plan.level_for(1, 2) == 1 and plan.choices is plan.levels
    b = lambda layer_id, dc, mc: None
    ft.register_block_builder(["AForCausalLM", "BForCausalLM"], b)
    ft.register_block_builder("AForCausalLM", b)                       # the same builder again: fine
    with pytest.raises(ValueError):
        ft.register_block_builder(["BForCausalLM"], lambda *a: None)


def test_more_reference_spellings(tmp_path):
    """Keyword names of the reference in the optimizers, exports, download helpers and FLOP helpers."""
    import pytest
    import torch
    import flextrain_b200 as ft
    from conftest import build_tiny
    from flextrain_b200.core.flop_accounting import bwd_flops, fwd_flops, opt_flops_per_step, step_flops
    from flextrain_b200.core._memory import get_available_gpu_memory
    from flextrain_b200.io.download import download_dataset, hf_checkpoint_is_complete, normalize_sft_record
    from flextrain_b200.optim import (AdamW, AdamWHyperparams, HybridMuonAdamW, HybridMuonAdamWHyperparams, Muon,
                                      MuonHyperparams, infer_optimizer_for_param)
    from flextrain_b200.core import TensorSpec
    a = AdamW(hp=AdamWHyperparams(lr=2e-4), state_dtype=torch.float32)
    assert a == AdamW(lr=2e-4, weight_decay=0.001, state_dtype=torch.float32)
    assert Muon(hp=MuonHyperparams(lr=5e-3)).lr == 5e-3
    h = HybridMuonAdamW(hp=HybridMuonAdamWHyperparams(lr=2e-3))
    assert h.muon.lr == h.adamw.lr == 2e-3 and h.adamw.state_dtype == torch.float32
    with pytest.raises(ValueError):
        MuonHyperparams(a=3.0)
    assert infer_optimizer_for_param(TensorSpec("w_q", (8, 8)), {}) == "muon"
    assert infer_optimizer_for_param(TensorSpec("w_router", (8, 8)), {}) == "adamw"
    assert infer_optimizer_for_param(TensorSpec("w_q", (8, 8), optimizer="adamw"), {}) == "adamw"
    # exports
    am = build_tiny(batch_tokens=512, lora_targets="all", lora_rank=4, lora_alpha=8.0)
    out = ft.export.save_hf_full(am, str(tmp_path / "full"), hf_source_dir=None, arch=None, shard_size_bytes=1 << 20)
    assert len([f for f in os.listdir(out) if f.endswith(".safetensors")]) > 1            # the small shard size took
    ad = ft.export.save_lora_adapter(am, str(tmp_path / "ad"), base_model_name_or_path="base", rank=4, alpha=8.0, bias="none")
    cfg = json.load(open(os.path.join(ad, "adapter_config.json")))
    assert cfg["r"] == 4 and cfg["lora_alpha"] == 8.0 and cfg["base_model_name_or_path"] == "base"
    for _, _, n, t in am.named_master_params():
        if n.endswith("_lora_b"):
            t.fill_(0.01)
    ft.export.save_hf_merged(am, str(tmp_path / "m1"))
    assert any(float(t.abs().max()) > 0 for _, _, n, t in am.named_master_params() if n.endswith("_lora_b"))
    ft.export.save_hf_merged(am, str(tmp_path / "m2"), keep_lora_after_merge=False)
    assert all(float(t.abs().max()) == 0 for _, _, n, t in am.named_master_params() if n.endswith("_lora_b"))
    assert ft.export.merge_lora_into_base(am) > 0
    # download helpers
    assert not hf_checkpoint_is_complete(tmp_path) and hf_checkpoint_is_complete(out)
    assert normalize_sft_record({"query": "q", "response": "r", "context": "c"}) == {"instruction": "q\nc", "response": "r"}
    src = tmp_path / "d.json"
    src.write_text(json.dumps([{"prompt": "p", "response": "r"}]))
    got = download_dataset(dataset_spec=str(src), target_path=str(tmp_path / "d.jsonl"), verbose=False)
    assert json.loads(open(got).readline())["instruction"] == "p"
    # FLOP helpers with a sequence length instead of recorded statistics
    plain = build_tiny(batch_tokens=512)
    seqs = ft.SyntheticTokenSource(1024, 128, seed=0).get_sequences(512)
    st = plain.fwd_bwd(seqs)
    head = 2.0 * 512 * plain.head.vocab_size * plain.head.d_model
    assert abs(4 * fwd_flops(plain, 128) - (st.fwd_flops + head)) < 1e-6 * st.fwd_flops
    assert bwd_flops(plain, 128, mode="lora") == fwd_flops(plain, 128) and bwd_flops(plain, 128) == 2 * fwd_flops(plain, 128)
    assert step_flops(plain, [128] * 4) == 12 * fwd_flops(plain, 128) + opt_flops_per_step(plain)
    assert get_available_gpu_memory("cpu") == get_available_gpu_memory(device="cpu") > 0


def test_an_optimizer_written_to_the_reference_protocol_trains_the_model():
    """``state_spec = OptimizerStateSpec(tensors=...)`` + ``step(..., *, step_num)``: SGD with momentum written that
    way drives the engine and matches ``torch.optim.SGD`` on the naive model."""
    import torch
    import flextrain_b200 as ft
    from conftest import build_tiny
    from flextrain_b200.bench.naive import clone_params, naive_loss
    from flextrain_b200.optim.base import Optimizer, OptimizerStateSpec, OptStateTensor  # noqa: F401

    class MomentumSGD:
        state_spec = OptimizerStateSpec(tensors=(OptStateTensor(name="o_buf", dtype=torch.float32),))

        def __init__(self, lr, mu):
            self.lr, self.mu, self.calls = lr, mu, []

        def step(self, param_spec, master, grads, state, *, step_num):
            self.calls.append(step_num)
            for p in param_spec.tensors:
                grad_key = "g_" + p.name[2:] if p.name.startswith("w_") else "g_" + p.name
                buf = state[f"o_buf_{p.name[2:] if p.name.startswith('w_') else p.name}"]
                buf.mul_(self.mu).add_(grads[grad_key].float())
                master[p.name].add_(buf.to(master[p.name].dtype), alpha=-self.lr)
            return 0

    opt = MomentumSGD(lr=0.05, mu=0.9)
    am = build_tiny(batch_tokens=256, optimizer=opt)
    P = clone_params(am)
    ref = torch.optim.SGD(list(P.values()), lr=0.05, momentum=0.9)
    src = ft.SyntheticTokenSource(1024, 128, seed=5)
    for step in range(3):
        seqs = src.get_sequences(256)
        st = am.fwd_bwd(seqs, loss_scale_factor=1.0 / 256)
        assert am.step() == 0
        ref.zero_grad()
        loss = naive_loss(am, P, seqs)                       # the mean over the 256 scored tokens
        loss.backward()
        ref.step()
        assert abs(st.loss_sum / 256 - float(loss)) < 2e-4
    assert opt.calls[:3] == [1, 1, 1] or opt.calls.count(3) >= 1          # called per unit, with the step number
    bm = am.buffers
    for (scope, l, name), p in P.items():
        mine = {"embed": bm.embed_params(), "head": bm.head_params()}.get(scope) or bm.host_params(l)
        torch.testing.assert_close(mine[name].float(), p.detach(), rtol=2e-4, atol=2e-5, msg=f"{scope}/{l}/{name}")
    am.optimizer.lr = 0.01
    assert opt.lr == 0.01


def test_duck_typed_sequences_are_accepted():
    """Any object with ``tokens`` (and optionally ``targets``, ``loss_mask``, ``seq_id``) is a sequence, as in the
    reference; per-token losses are written back to the caller's own objects."""
    import pytest
    import torch
    import flextrain_b200 as ft
    from conftest import build_tiny

    class Mine:
        def __init__(self, tokens):
            self.tokens = tokens
            self.targets = torch.roll(tokens, -1)
            self.per_token_loss = torch.zeros(len(tokens))
            self.seq_id = 0

        def __len__(self):
            return len(self.tokens)

    g = torch.Generator().manual_seed(0)
    toks = [torch.randint(0, 1024, (100,), generator=g), torch.randint(0, 1024, (60,), generator=g)]
    mine = [Mine(t) for t in toks]
    mine[0].targets[:10] = -100
    theirs = [ft.Sequence(t.clone(), targets=m.targets.clone()) for t, m in zip(toks, mine)]
    a, b = build_tiny(batch_tokens=256), build_tiny(batch_tokens=256)
    sa = a.fwd_bwd(mine, loss_scale_factor=1.0 / 150)
    sb = b.fwd_bwd(theirs, loss_scale_factor=1.0 / 150)
    assert sa.loss_sum == sb.loss_sum and sa.active_tokens == 150
    assert float(mine[0].per_token_loss[:10].abs().max()) == 0 and float(mine[0].per_token_loss[10]) > 0
    assert torch.equal(mine[1].per_token_loss, theirs[1].per_token_loss)
    with pytest.raises(TypeError):
        a.fwd_bwd([object()])


def test_sequences_are_checked_on_the_host_before_anything_reaches_the_device():
    """Too long for the context window, a token id outside the embedding table, a target that is neither a vocabulary
    id nor the ignore value, an empty sequence: each is a ``ValueError`` at the call, not an out-of-range access later."""
    import pytest
    import torch
    import flextrain_b200 as ft
    from conftest import build_tiny
    am = build_tiny(batch_tokens=256, max_seq_len=128)
    ids = lambda n, v=0: torch.full((n,), v, dtype=torch.int64)
    bad_target = ids(16)
    bad_target[3] = -1
    for seq, what in [(ft.Sequence(ids(200)), "max_seq_len=128"), (ft.Sequence(ids(16, 5000)), "token id 5000"),
                      (ft.Sequence(ids(16, -1)), "token id -1"), (ft.Sequence(ids(16), targets=bad_target), "target outside"),
                      (ft.Sequence(ids(16), targets=ids(16, 1024)), "target outside"), (ft.Sequence(ids(0)), "is empty"),
                      (ft.Sequence(ids(16), targets=ids(8)), "8 targets for 16 tokens"),
                      (ft.Sequence(ids(16), loss_mask=torch.ones(4)), "4 loss_mask entries"),
                      (ft.Sequence(ids(16), advantages=torch.ones(20)), "20 advantages entries")]:
        with pytest.raises(ValueError, match=what):
            am.fwd_bwd([seq])
        with pytest.raises(ValueError, match=what):
            am.evaluate([seq])
    ok = ft.Sequence(ids(16, 1023), targets=torch.full((16,), -100, dtype=torch.int64))
    assert am.fwd_bwd([ok]).active_tokens == 0
