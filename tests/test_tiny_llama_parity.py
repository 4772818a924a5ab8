"""Tiny Llama on CPU in fp32: the engine's hand-written forward/backward/optimizer against
``torch.autograd`` + ``torch.optim.AdamW`` (2 layers, hidden 256, 4 query / 2 KV heads, head_dim 64,
SwiGLU 688, vocab 1024, seq 128, batch 2, 3 AdamW steps at lr 1e-3)."""
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
