"""Tiny Llama on CPU in fp32: the engine's hand-written forward/backward/optimizer against
``torch.autograd`` + ``torch.optim.AdamW`` (2 layers, hidden 256, 4 query / 2 KV heads, head_dim 64,
SwiGLU 688, vocab 1024, seq 128, batch 2, 3 AdamW steps at lr 1e-3)."""
import pytest
import torch

import flextrain_b200 as ft
from flextrain_b200.bench.naive import clone_params, naive_loss
from conftest import build_tiny


def _seqs(n=2, L=128, seed=0, vocab=1024):
    src = ft.SyntheticTokenSource(vocab, L, seed=seed)
    return src.get_sequences(n * L)


def test_forward_backward_matches_autograd():
    am = build_tiny()
    seqs = _seqs()
    P = clone_params(am)
    loss = naive_loss(am, P, seqs)
    loss.backward()
    st = am.fwd_bwd(seqs)
    assert abs(st.loss - float(loss)) < 1e-4
    bm = am.buffers
    checked = 0
    for (scope, l, name), p in P.items():
        gname = "g_" + name[2:]
        g = {"embed": bm.embed_grads(), "head": bm.head_grads()}.get(scope) or bm.grads(l)
        torch.testing.assert_close(g[gname].float(), p.grad, rtol=2e-4, atol=2e-6, msg=f"{scope}/{l}/{name}")
        checked += 1
    assert checked == 2 * 9 + 3


def test_three_adamw_steps_track_torch_optim():
    am = build_tiny()
    P = clone_params(am)
    opt = torch.optim.AdamW(list(P.values()), lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0)
    src = ft.SyntheticTokenSource(1024, 128, seed=1)
    for step in range(3):
        seqs = src.get_sequences(256)
        opt.zero_grad()
        loss = naive_loss(am, P, seqs)
        loss.backward()
        opt.step()
        st = am.fwd_bwd(seqs)
        assert am.step() == 0
        assert abs(st.loss - float(loss)) < 2e-4, (step, st.loss, float(loss))
    for scope, l, name, t in am.named_master_params():
        # Adam turns a near-zero gradient into a +-lr step, so single elements may differ by ~lr; the bulk must agree
        d = (t.float() - P[(scope, l, name)].detach()).abs()
        assert float(d.max()) < 2.5e-3 and float(d.mean()) < 2e-6, (scope, l, name, float(d.max()), float(d.mean()))


def test_per_token_loss_written_back():
    am = build_tiny()
    seqs = _seqs()
    st = am.fwd_bwd(seqs)
    tot = sum(float(s.per_token_loss.sum()) for s in seqs)
    assert abs(tot - st.loss_sum) < 1e-2
    assert st.active_tokens == 256 and st.tokens == 256


@pytest.mark.parametrize("tied", [False, True])
def test_gradient_accumulation_over_calls_equals_one_call(tied):
    """Gradients accumulate over ``fwd_bwd`` calls until ``step``: two calls with half the batch each (and the whole
    batch's scale factor) leave the same weights as one call with everything — also for tied embeddings, whose
    head share is folded into the embedding gradient at the end of every call."""
    import flextrain_b200 as ft
    from conftest import build_tiny
    dims = dict(vocab_size=256, n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, expert_dim=128,
                ffn_dim=128, num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)
    mk = lambda: build_tiny(dims=dims, hyper={"tie_embeddings": tied}, max_seq_len=64, batch_tokens=256,
                            optimizer=ft.AdamW(lr=1e-3, state_dtype=torch.float32))
    seqs = ft.SyntheticTokenSource(256, 64, seed=7).get_sequences(256)
    n_active = sum(s.active_token_count for s in seqs)
    a, b = mk(), mk()
    assert a.head.tied == tied
    a.fwd_bwd(seqs, loss_scale_factor=1.0 / n_active)
    a.step()
    b.fwd_bwd(seqs[:2], loss_scale_factor=1.0 / n_active)
    b.fwd_bwd(seqs[2:], loss_scale_factor=1.0 / n_active)
    b.step()
    for (s, l, n, t), (_, _, _, u) in zip(a.named_master_params(), b.named_master_params()):
        torch.testing.assert_close(t, u, rtol=0, atol=2e-6, msg=f"{s}/{l}/{n}")
    if tied:
        assert torch.equal(a.buffers.head_params()["w_head_proj"], a.buffers.embed_params()["w_tok_embeddings"])


@pytest.mark.parametrize("rings", [False, True])
def test_gradient_clipping_tracks_torch(rings):
    """``am.step(max_grad_norm=c)``: the reported global norm equals ``torch.nn.utils.clip_grad_norm_``'s and three
    clipped AdamW steps follow torch's (resident state, and with weight / gradient / optimizer rings)."""
    kw = {}
    if rings:
        kw["ws"] = ft.WorkingSetConfig.simple(max_seq_len=128, max_global_batch_tokens=256, n_gpu_layers=1, n_gpu_grads=1,
                                              n_gpu_opt_layers=1)
    am = build_tiny(**kw)
    P = clone_params(am)
    opt = torch.optim.AdamW(list(P.values()), lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0)
    src = ft.SyntheticTokenSource(1024, 128, seed=1)
    clip = 0.3
    for step in range(3):
        seqs = src.get_sequences(256)
        opt.zero_grad()
        loss = naive_loss(am, P, seqs)
        loss.backward()
        want_norm = float(torch.nn.utils.clip_grad_norm_(list(P.values()), clip))
        opt.step()
        st = am.fwd_bwd(seqs)
        assert am.step(max_grad_norm=clip) == 0
        assert want_norm > clip                                             # the clip is active
        assert abs(am.last_grad_norm - want_norm) < 1e-4 * want_norm, (step, am.last_grad_norm, want_norm)
        assert abs(st.loss - float(loss)) < 2e-4, (step, st.loss, float(loss))
    for scope, l, name, t in am.named_master_params():
        d = (t.float() - P[(scope, l, name)].detach()).abs()
        assert float(d.max()) < 2.5e-3 and float(d.mean()) < 2e-6, (scope, l, name, float(d.max()), float(d.mean()))
