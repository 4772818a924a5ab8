"""Property-based checks (hypothesis) of the host-side bookkeeping that everything else leans on: chunk packing, round
splitting, chunk padding, data-parallel shard ranges, the splice maps and the image resize rule."""
import math

import pytest
import torch

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import given, settings, strategies as st  # noqa: E402

import flextrain_b200 as ft  # noqa: E402
from flextrain_b200.engine.schedule import pack_sequences, prepare_training_chunks, split_sequences  # noqa: E402
from flextrain_b200.io.image_processing import smart_resize  # noqa: E402
from flextrain_b200.nn.splices.concat import build_splice_maps  # noqa: E402
from flextrain_b200.parallel.dp import shard_range  # noqa: E402

lens_st = st.lists(st.integers(1, 700), min_size=1, max_size=12)


def _seqs(lens, vocab=50):
    g = torch.Generator().manual_seed(sum(lens))
    return [ft.Sequence(torch.randint(0, vocab, (n,), generator=g), seq_id=i) for i, n in enumerate(lens)]


@settings(max_examples=60, deadline=None)
@given(lens=lens_st, chunk=st.sampled_from([64, 128, 200, 256, 512]))
def test_packing_covers_every_token_once_in_order(lens, chunk):
    seqs = _seqs(lens)
    plans = pack_sequences(seqs, chunk)
    seen = {i: 0 for i in range(len(seqs))}
    last_seq = -1
    for p in plans:
        assert 0 < p.num_tokens <= chunk
        for i, start, n in p.pieces:
            assert start == seen[i] and n > 0 and i >= last_seq          # contiguous, in order
            seen[i] += n
            last_seq = i
        if any(start > 0 or start + n < len(seqs[i]) for i, start, n in p.pieces):
            assert len(p.pieces) == 1                                    # a split sequence never shares its chunks
    assert all(seen[i] == len(s) for i, s in enumerate(seqs))
    # chunks of one sequence group are consecutive and groups only grow
    assert [p.seq_group for p in plans] == sorted(p.seq_group for p in plans)


@settings(max_examples=60, deadline=None)
@given(lens=lens_st, chunk=st.sampled_from([128, 256]), target=st.sampled_from([256, 512, 1024]))
def test_rounds_hold_whole_sequences_in_order(lens, chunk, target):
    seqs = _seqs(lens)
    rounds = split_sequences(seqs, target_round_tokens=target, max_chunk_size=chunk, max_training_chunks=64,
                             max_total_round_tokens=max(target, 1024))
    flat = [s.seq_id for r in rounds for s in r]
    assert flat == [s.seq_id for s in seqs]
    for r in rounds:
        tot = sum(len(s) for s in r)
        assert tot <= max(target, 1024) and (len(r) == 1 or tot <= target)


@settings(max_examples=40, deadline=None)
@given(lens=st.lists(st.integers(1, 250), min_size=1, max_size=8), mult=st.sampled_from([128, 256]))
def test_padded_chunks_keep_the_real_tokens_and_score_none_of_the_filler(lens, mult):
    seqs = _seqs(lens)
    plain = prepare_training_chunks(seqs, 256, "cpu")
    padded = prepare_training_chunks(seqs, 256, "cpu", pad_multiple=mult)
    assert len(plain) == len(padded)
    for a, b in zip(plain, padded):
        pad = b.extra["pad_tokens"]
        assert b.num_tokens % mult == 0 and b.num_tokens == a.num_tokens + pad and 0 <= pad < mult
        assert torch.equal(a.tokens, b.tokens[: a.num_tokens]) and torch.equal(a.targets, b.targets[: a.num_tokens])
        assert torch.equal(a.positions, b.positions[: a.num_tokens])
        assert bool((b.targets[a.num_tokens:] == -100).all())
        assert a.seq_lens[:-1] == b.seq_lens[:-1] and b.seq_lens[-1] == a.seq_lens[-1] + pad


@settings(max_examples=100, deadline=None)
@given(n=st.integers(0, 10 ** 7), world=st.integers(1, 8))
def test_shard_ranges_partition_the_elements(n, world):
    pos = 0
    for r in range(world):
        b, c = shard_range(n, r, world)
        assert b == pos and c >= 0
        pos += c
    assert pos == n


@settings(max_examples=60, deadline=None)
@given(h=st.integers(8, 3000), w=st.integers(8, 3000), factor=st.sampled_from([8, 28, 32]))
def test_smart_resize_rule(h, w, factor):
    lo, hi = 56 * 56, 28 * 28 * 1280
    if max(h, w) / min(h, w) > 200:
        return
    H, W = smart_resize(h, w, factor, lo, hi)
    assert H % factor == 0 and W % factor == 0 and H >= factor and W >= factor
    assert H * W <= hi
    assert H * W >= lo or (H, W) == (max(factor, math.ceil(h * math.sqrt(lo / (h * w)) / factor) * factor),
                                     max(factor, math.ceil(w * math.sqrt(lo / (h * w)) / factor) * factor))
    if lo <= round(h / factor) * factor * round(w / factor) * factor <= hi:
        assert abs(H - h) <= factor / 2 and abs(W - w) <= factor / 2     # nearest multiples when the area allows


@settings(max_examples=40, deadline=None)
@given(data=st.data())
def test_splice_maps_place_every_image_row_once(data):
    n_seq = data.draw(st.integers(1, 4))
    PH = 9
    seqs, offsets, acc = [], {}, 0
    for i in range(n_seq):
        n = data.draw(st.integers(4, 120))
        toks = torch.tensor(data.draw(st.lists(st.sampled_from([1, 2, PH]), min_size=n, max_size=n)))
        seqs.append(ft.Sequence(toks, seq_id=i))
        k = int((toks == PH).sum())
        if k:
            offsets[i] = acc
            acc += k
    chunk = data.draw(st.sampled_from([16, 32, 64]))
    plans = pack_sequences(seqs, chunk)
    maps = build_splice_maps(seqs, [p.pieces for p in plans], [PH], offsets)
    used = []
    for p, m in zip(plans, maps):
        toks = torch.cat([seqs[i].tokens[s:s + n] for i, s, n in p.pieces])
        rows = (toks == PH).nonzero(as_tuple=True)[0]
        if m is None:
            assert rows.numel() == 0
            continue
        assert torch.equal(m[0], rows)
        used += m[1].tolist()
    assert used == list(range(acc))                        # in order, each encoder row exactly once
