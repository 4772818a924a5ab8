"""Pluggable losses (GRPO with per-token advantages and a KL penalty to reference log-probs, MSE) through the whole
engine on CPU: the in-place ``dZ`` each loss writes must reproduce autograd's gradients of the same formula on the naive
model (the reference: flextrain/nn/loss.py:68-442)."""
import pytest
import torch

import flextrain_b200 as ft
from flextrain_b200.bench.naive import clone_params, naive_forward
from flextrain_b200.nn.loss import GRPOLoss, MSELoss
from conftest import build_tiny

DIMS = dict(vocab_size=256, n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, expert_dim=128, ffn_dim=128,
            num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)


def _seqs():
    g = torch.Generator().manual_seed(0)
    out = []
    for i, n in enumerate((40, 24)):
        t = torch.randint(0, 256, (n,), generator=g)
        tgt = torch.roll(t, -1)
        tgt[-1] = -100
        tgt[:3] = -100                                         # a prompt that is not trained on
        out.append(ft.Sequence(t, targets=tgt, seq_id=i, advantages=torch.randn(n, generator=g),
                               ref_logprobs=-5.0 + torch.randn(n, generator=g) * 0.3))
    return out


def _compare(am, P, loss):
    loss.backward()
    bm = am.buffers
    n = 0
    for (scope, l, name), p in P.items():
        g = {"embed": bm.embed_grads(), "head": bm.head_grads()}.get(scope) or bm.grads(l)
        gname = "g_" + name[2:] if name.startswith("w_") else "g_" + name
        if gname in g and p.grad is not None:
            torch.testing.assert_close(g[gname].float(), p.grad, rtol=3e-4, atol=3e-6, msg=f"{scope}/{l}/{name}")
            n += 1
    assert n > 5


@pytest.mark.parametrize("beta", [0.0, 0.2])
def test_grpo_loss_gradients(beta):
    am = build_tiny(dims=DIMS, max_seq_len=48, batch_tokens=96)
    seqs = _seqs()
    P = clone_params(am)
    total, per_tok = 0.0, []
    for s in seqs:
        logp = torch.log_softmax(naive_forward(am, P, s.tokens), -1)
        valid = (s.targets != -100)
        lp = logp.gather(1, s.targets.clamp(min=0)[:, None])[:, 0]
        li = -s.advantages * lp
        if beta:
            d = s.ref_logprobs - lp
            li = li + beta * (torch.exp(d) - d - 1)             # k3 estimator of KL(pi || ref) on the taken token
        total = total + (li * valid).sum()
        per_tok.append((li * valid).detach())
    st = am.fwd_bwd(seqs, loss_scale_factor=1.0, loss_fn=GRPOLoss(kl_beta=beta))
    assert abs(st.loss_sum - float(total)) < 1e-3 * max(1.0, abs(float(total)))
    _compare(am, P, total)
    for s, want in zip(seqs, per_tok):                          # per-token losses are written back to the sequences
        torch.testing.assert_close(s.per_token_loss[: len(s)].float(), want, rtol=1e-4, atol=1e-5)


def test_mse_loss_gradients():
    am = build_tiny(dims=DIMS, max_seq_len=48, batch_tokens=96)
    seqs = _seqs()
    P = clone_params(am)
    total = 0.0
    for s in seqs:
        z = naive_forward(am, P, s.tokens)
        valid = (s.targets != -100)
        onehot = torch.nn.functional.one_hot(s.targets.clamp(min=0), z.shape[1]).to(z.dtype)
        total = total + (((z - onehot) ** 2).mean(-1) * valid).sum()
    st = am.fwd_bwd(seqs, loss_scale_factor=1.0, loss_fn=MSELoss())
    assert abs(st.loss_sum - float(total)) < 1e-3 * max(1.0, abs(float(total)))
    _compare(am, P, total)


class _RefStyleLabelSmoothing:
    """A loss written against the reference's protocol: ``compute`` returns UNscaled ``dZ`` and fills
    ``per_token_loss_out``; it reads ``token_slice.labels``."""

    def __init__(self, eps):
        self.eps = eps

    def compute(self, logits, token_slice, *, loss_scale, per_token_loss_out):
        z = logits.to(torch.float32)
        labels = token_slice.labels
        valid = labels != -100
        logp = torch.log_softmax(z, -1)
        V = z.shape[1]
        target = torch.full_like(z, self.eps / V)
        target.scatter_(1, labels.clamp(min=0).long().unsqueeze(1), 1.0 - self.eps + self.eps / V)
        per_token_loss_out.copy_(-(target * logp).sum(-1) * valid)
        dz = (torch.exp(logp) - target) * valid.unsqueeze(1)
        return dz.to(logits.dtype), {"smoothing": self.eps}


@pytest.mark.parametrize("softcap", [0.0, 5.0])
def test_reference_style_loss_object_matches_autograd(softcap):
    """A ``compute``-style loss (the reference's protocol) runs through the engine; with a final soft-cap the loss
    sees capped logits and its gradient is carried back through the cap."""
    am = build_tiny(dims=DIMS, max_seq_len=48, batch_tokens=96)
    seqs = _seqs()
    eps = 0.1
    am.head.final_softcap = softcap
    st = am.fwd_bwd(seqs, loss_scale_factor=0.5, loss_fn=_RefStyleLabelSmoothing(eps))
    am.head.final_softcap = 0.0                      # the naive forward below applies the cap itself
    P = clone_params(am)
    total = 0.0
    for s in seqs:
        z = naive_forward(am, P, s.tokens).float()
        if softcap:
            z = softcap * torch.tanh(z / softcap)
        logp = torch.log_softmax(z, -1)
        valid = s.targets != -100
        V = z.shape[1]
        target = torch.full_like(z, eps / V)
        target.scatter_(1, s.targets.clamp(min=0).unsqueeze(1), 1.0 - eps + eps / V)
        total = total + (-(target * logp).sum(-1) * valid).sum()
    assert abs(st.loss_sum - float(total)) < 1e-3 * float(total)
    _compare(am, P, total * 0.5)


def test_builtin_losses_answer_to_the_reference_call_and_names():
    from flextrain_b200.nn.loss import CrossEntropyLoss, TokenContext, TokenSlice
    torch.manual_seed(0)
    z = torch.randn(6, 11)
    labels = torch.tensor([1, 2, -100, 4, 5, 6])
    ctx = TokenContext(labels=labels, advantages=torch.ones(6))
    sl = ctx.slice_for(2, 4)
    assert sl.offset == 2 and sl.size == 4 and sl.labels is sl.targets and sl.targets.tolist() == [-100, 4, 5, 6]
    assert ctx.total_tokens == 6 and TokenSlice(labels=labels).targets is labels
    out = torch.empty(6)
    zz = z.clone()
    dz, aux = CrossEntropyLoss(ignore_index=-100).compute(zz, TokenSlice(labels), loss_scale=0.25, per_token_loss_out=out)
    want = torch.nn.functional.cross_entropy(z, labels, ignore_index=-100, reduction="none")
    torch.testing.assert_close(out, want)
    p = torch.softmax(z, -1)
    onehot = torch.zeros_like(p).scatter_(1, labels.clamp(min=0).unsqueeze(1), 1.0)
    torch.testing.assert_close(dz, (p - onehot) * (labels != -100).unsqueeze(1))       # unscaled, as the reference says
    assert GRPOLoss(kl_coef=0.3).kl_beta == 0.3
