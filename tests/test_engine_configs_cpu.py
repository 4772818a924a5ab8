"""Engine scheduling paths forced by hand-built working sets (the reference's parity harness configs A-H,
flextrain/bench/README.md:45-66): A all-on-device, B multi-chunk, C multi-round, D host offload at each tier,
E weight ring, F grad ring, G opt ring, H a sequence that spans chunks.  The plan changes where tensors live,
never what is computed, so losses and updated weights must agree with config A to fp32 round-off."""
import pytest
import torch

import flextrain_b200 as ft
from flextrain_b200.bench.naive import clone_params, naive_loss
from conftest import build_tiny

DIMS = dict(vocab_size=512, n_layers=4, d_model=128, n_heads=4, n_kv_heads=2, head_dim=32, expert_dim=256, ffn_dim=256,
            num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)


def _run(ws_kw=None, steps=2, seq_lens=(64, 48, 64, 80), force=None, arch="llama", dims=DIMS, hyper=None, max_seq=96):
    ws = ft.WorkingSetConfig.simple(max_seq_len=max_seq, max_global_batch_tokens=256, **(ws_kw or {}))
    am = build_tiny(arch=arch, dims=dims, hyper=hyper, ws=ws, max_seq_len=max_seq, batch_tokens=256,
                    force_saved_act_level=force)
    src = ft.SyntheticTokenSource(dims["vocab_size"], list(seq_lens), seed=4)
    losses = []
    for _ in range(steps):
        seqs = src.get_sequences(256)
        st = am.fwd_bwd(seqs)
        assert am.step() == 0
        losses.append(st.loss)
    flat = torch.cat([t.flatten().float() for _, _, _, t in am.named_master_params()])
    return losses, flat, am


@pytest.fixture(scope="module")
def base():
    return _run()


def _same(a, b, tol=2e-5):
    for x, y in zip(a[0], b[0]):
        assert abs(x - y) < 1e-4, (a[0], b[0])
    d = (a[1] - b[1]).abs()
    assert float(d.mean()) < tol and float(d.max()) < 2.5e-3, (float(d.mean()), float(d.max()))


def test_B_multi_chunk(base):
    _same(base, _run(dict(chunk=96)))


def test_C_multi_round(base):
    r = _run(dict(chunk=96, round_tokens=128))
    assert r[2].ws.target_num_rounds >= 2
    _same(base, r)


@pytest.mark.parametrize("level", [0, 1, 2, 3])
def test_D_forced_save_level_with_host_offload(base, level):
    r = _run(dict(chunk=96, host_act_buffer_size=64 << 20), force=level)
    assert set(r[2]._last_plan.histogram()) == {level}
    _same(base, r)


def test_D_solver_plan_with_few_device_slots(base):
    r = _run(dict(chunk=96, host_act_buffer_size=64 << 20, n_gpu_act_slots=3))
    hist = r[2]._last_plan.histogram()
    assert any(k >= 0 for k in hist), hist
    _same(base, r)


def test_E_weight_ring(base):
    _same(base, _run(dict(n_gpu_layers=2)))


def test_F_grad_ring(base):
    _same(base, _run(dict(n_gpu_grads=2, chunk=96, round_tokens=128)))


def test_G_opt_ring(base):
    _same(base, _run(dict(n_gpu_opt_layers=2)))


def test_EFG_all_rings_multi_round(base):
    r = _run(dict(n_gpu_layers=2, n_gpu_grads=2, n_gpu_opt_layers=2, chunk=96, round_tokens=128))
    _same(base, r)
    nbytes, ncopies = r[2]._ce.stats()          # the ring transfers went through the C++ copy engine
    assert ncopies > 0 and nbytes > 0


def test_copy_engine_can_be_switched_off(base, monkeypatch):
    monkeypatch.setenv("FTB_COPY_ENGINE", "0")
    r = _run(dict(n_gpu_layers=2, chunk=96, host_act_buffer_size=64 << 20), force=1)
    assert r[2]._ce is None
    monkeypatch.delenv("FTB_COPY_ENGINE")
    r2 = _run(dict(n_gpu_layers=2, chunk=96, host_act_buffer_size=64 << 20), force=1)
    assert r2[2]._ce is not None and r2[2]._ce.stats()[1] > 0
    _same(r, r2)


def test_H_sequence_spans_chunks_matches_autograd():
    ws = ft.WorkingSetConfig.simple(max_seq_len=160, max_global_batch_tokens=256, chunk=64)
    am = build_tiny(dims=DIMS, ws=ws, max_seq_len=160, batch_tokens=256)
    seqs = ft.SyntheticTokenSource(512, [150, 40, 66], seed=9).get_sequences(256)
    P = clone_params(am)
    loss = naive_loss(am, P, seqs)
    loss.backward()
    st = am.fwd_bwd(seqs)
    assert st.n_chunks >= 5
    assert abs(st.loss - float(loss.detach())) < 2e-4
    for (scope, l, name), p in P.items():
        g = {"embed": am.buffers.embed_grads(), "head": am.buffers.head_grads()}.get(scope) or am.buffers.grads(l)
        torch.testing.assert_close(g["g_" + name[2:]].float(), p.grad, rtol=3e-4, atol=3e-6, msg=f"{scope}/{l}/{name}")


def test_H_hybrid_linear_attention_spans_chunks():
    dims = dict(DIMS, n_layers=2)
    hyper = {"layer_pattern": "1L1F", "gdn": {"n_k_heads": 2, "n_v_heads": 2, "head_k_dim": 16, "head_v_dim": 32}}
    ws = ft.WorkingSetConfig.simple(max_seq_len=100, max_global_batch_tokens=128, chunk=32)
    am = build_tiny(arch="qwen3_5", dims=dims, hyper=hyper, ws=ws, max_seq_len=100, batch_tokens=128)
    seqs = ft.SyntheticTokenSource(512, [90, 30], seed=10).get_sequences(128)
    P = clone_params(am)
    loss = naive_loss(am, P, seqs)
    loss.backward()
    st = am.fwd_bwd(seqs)
    assert abs(st.loss - float(loss.detach())) < 2e-4, (st.loss, float(loss))
    for (scope, l, name), p in P.items():
        g = {"embed": am.buffers.embed_grads(), "head": am.buffers.head_grads()}.get(scope) or am.buffers.grads(l)
        gname = "g_" + name[2:]
        if gname in g:
            torch.testing.assert_close(g[gname].float(), p.grad, rtol=5e-4, atol=5e-6, msg=f"{scope}/{l}/{name}")


@pytest.mark.parametrize("variant", ["resident", "rings_and_host_acts", "multi_chunk_sequence"])
def test_evaluate_is_forward_only(variant):
    """``am.evaluate`` returns the loss ``fwd_bwd`` would, leaves accumulated gradients, optimizer state and the step
    counter alone, and a training run with evaluations in between equals one without."""
    import flextrain_b200 as ft
    dims = dict(vocab_size=256, n_layers=3, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, expert_dim=128,
                ffn_dim=128, num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)
    kw = dict(dims=dims, max_seq_len=128, batch_tokens=256, optimizer=ft.AdamW(lr=2e-3, state_dtype=torch.float32))
    if variant == "rings_and_host_acts":
        kw["ws"] = ft.WorkingSetConfig.simple(max_seq_len=128, max_global_batch_tokens=256, chunk=64, n_gpu_layers=2,
                                              n_gpu_grads=2, n_gpu_opt_layers=2, host_act_buffer_size=64 << 20,
                                              n_gpu_act_slots=2)
    if variant == "multi_chunk_sequence":
        kw["ws"] = ft.WorkingSetConfig.simple(max_seq_len=128, max_global_batch_tokens=256, chunk=32)
    src = lambda seed: ft.SyntheticTokenSource(256, 128, seed=seed)
    a, b = build_tiny(**kw), build_tiny(**kw)
    train, held_out = src(1), src(2).get_sequences(256)
    la, lb = [], []
    for step in range(3):
        seqs = train.get_sequences(256)
        half = a.fwd_bwd(seqs[:1], loss_scale_factor=1.0 / 256)            # gradients pending ...
        g_before = a.buffers.grads(1)["g_q"].clone() if a.buffers.grads_resident else None
        ev = a.evaluate(held_out)                                           # ... while an evaluation runs
        if g_before is not None:
            assert torch.equal(a.buffers.grads(1)["g_q"], g_before)
        rest = a.fwd_bwd(seqs[1:], loss_scale_factor=1.0 / 256)
        assert a.step() == 0 and a.step_num == step + 1
        la.append((half.loss_sum + rest.loss_sum) / 256)
        st = b.fwd_bwd(seqs, loss_scale_factor=1.0 / 256)
        assert b.step() == 0
        lb.append(st.loss_sum / 256)
        # the evaluation saw the same weights b had before this step: compare with b's own forward+backward on them
        assert ev.active_tokens == sum(s.active_token_count for s in held_out) and ev.loss > 0
    assert max(abs(x - y) for x, y in zip(la, lb)) < 1e-6, (la, lb)
    for (_, _, n, t), (_, _, _, u) in zip(a.named_master_params(), b.named_master_params()):
        torch.testing.assert_close(t, u, rtol=0, atol=1e-6, msg=n)
    want = b.fwd_bwd(held_out, loss_scale_factor=1.0)                       # same weights now: same loss as evaluate
    b._zero_grad = True
    assert abs(a.evaluate(held_out).loss_sum - want.loss_sum) < 1e-3
    assert held_out[0].per_token_loss is not None


# ------------------------------------------------------------------ stream-protocol checker
RINGS = dict(n_gpu_layers=2, n_gpu_grads=2, n_gpu_opt_layers=2, chunk=96, round_tokens=128)


def test_protocol_checker_passes_the_ring_schedules(monkeypatch):
    """With ``FTB_STREAM_CHECK=1`` every ring-slot access of the weight / gradient / optimizer rings (forward,
    backward over several rounds, streamed optimizer step) and of the K/V window of a sequence that spans chunks is
    replayed through vector clocks: the engine's events must order every write after the accesses it conflicts with."""
    monkeypatch.setenv("FTB_STREAM_CHECK", "1")
    _, _, am = _run(RINGS)
    chk = am.streams.checker
    assert chk is not None and chk.n_accesses > 50
    assert {k[0] for k in chk.history} >= {"p", "g", "o"}
    assert am.protocol_violations() == []
    _, _, am2 = _run(dict(chunk=64), seq_lens=(160, 96), max_seq=160)          # sequences that span chunks
    assert ("kv",) in am2.streams.checker.history and am2.protocol_violations() == []


@pytest.mark.parametrize("dropped", ["layer_out", "weights_in", "opt_in"])
def test_protocol_checker_catches_a_missing_wait(monkeypatch, dropped):
    """Take one class of waits out of the schedule (the copy that refills a ring slot no longer waits for the layer
    that used it / compute no longer waits for its weights / the update no longer waits for its state): nothing
    crashes, the run even finishes, and the checker names the unordered access."""
    from flextrain_b200.engine import streams as S
    monkeypatch.setenv("FTB_STREAM_CHECK", "1")
    real = S.EventMap.wait

    def wait(self, key, stream):
        if self.name == dropped:
            if key not in self._ev:
                raise KeyError(key)
            return None                      # the scheduling bug: the wait is simply not issued
        return real(self, key, stream)

    monkeypatch.setattr(S.EventMap, "wait", wait)
    _, _, am = _run(RINGS, steps=1)
    v = am.protocol_violations()
    assert v, "a dropped wait must be reported"
    kinds = {"layer_out": "write-after-read", "weights_in": "read-after-write", "opt_in": "after-write"}
    assert any(kinds[dropped] in s for s in v), v[:3]
