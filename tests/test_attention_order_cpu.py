"""The ordered-dQ protocol of the attention backward, checked on the host.

The kernel (``csrc/attention.cu::fa_bwd_kernel``) runs one CTA per key tile; with the ordered mode on, the CTA of key
tile ``j`` adds its share of a query tile's dQ only after the key tiles above ``j`` that touch that query tile have
added theirs (one counter per (query tile, head)).  Blocks are handed out in increasing ``blockIdx``, and only as many
run at once as fit on the GPU, so the mapping block -> key tile must make every CTA wait only for CTAs that were handed
out before it.  This test restates the kernel's index arithmetic and replays the protocol with a small number of
resident CTAs over random ragged batches (prior context, sliding windows, non-causal): it must finish without a
wait that can never be satisfied, every counter must end at the number of key tiles that touch its query tile, and the
additions to a query tile must come in strictly descending key-tile order."""
import random

import pytest

TQ = 128


def ctas_in_dispatch_order(lens_q, lens_k, causal, window, rep, grid_slack=3):
    """[(seq, k0, iterations)] in blockIdx order for one KV head; an iteration is (counter key, expected, key tile)."""
    n_tiles = [(lk + TQ - 1) // TQ for lk in lens_k]
    grid = sum(n_tiles) + grid_slack                  # the host passes an upper bound of the tile count
    qtile_base, acc = [], 0
    for lq in lens_q:
        qtile_base.append(acc)
        acc += (lq + TQ - 1) // TQ
    out = []
    for block in range(grid):
        tile = grid - 1 - block                       # ordered mode: descending key tiles
        seq, a = None, 0
        for s, nt in enumerate(n_tiles):
            if tile < a + nt:
                seq, k0 = s, (tile - a) * TQ
                break
            a += nt
        if seq is None:
            continue                                  # block beyond the real tile count: exits at once
        len_q, len_k = lens_q[seq], lens_k[seq]
        off = len_k - len_q
        kr = min(TQ, len_k - k0)
        i_lo = max(0, k0 - off) if causal else 0
        i_hi = min(len_q, k0 + kr + window - 1 - off) if (causal and window > 0) else len_q
        i_lo = (i_lo // TQ) * TQ
        n_qt = (i_hi - i_lo + TQ - 1) // TQ if i_hi > i_lo else 0
        n_kt = (len_k + TQ - 1) // TQ
        its = []
        for it in range(n_qt * rep):
            h, qt = it // n_qt, i_lo + (it % n_qt) * TQ
            j_hi = min(n_kt - 1, (qt + TQ - 1 + off) // TQ) if causal else n_kt - 1
            its.append(((qtile_base[seq] + qt // TQ, h), j_hi - k0 // TQ, k0 // TQ))
        out.append((seq, k0, its))
    return out


def replay(ctas, resident):
    """Run the CTAs ``resident`` at a time in dispatch order; returns (finished, counters, per-counter add order)."""
    sem, order = {}, {}
    waiting = list(range(len(ctas)))
    running = {}                                      # cta index -> next iteration
    while waiting or running:
        while waiting and len(running) < resident:
            running[waiting.pop(0)] = 0
        progressed = False
        for c in sorted(running):
            its = ctas[c][2]
            while running[c] < len(its):
                key, expected, jt = its[running[c]]
                if sem.get(key, 0) < expected:
                    break
                sem[key] = sem.get(key, 0) + 1
                order.setdefault(key, []).append(jt)
                running[c] += 1
                progressed = True
            if running[c] == len(its):
                del running[c]
                progressed = True
        if not progressed:
            return False, sem, order
    return True, sem, order


@pytest.mark.parametrize("seed", range(12))
def test_ordered_dq_never_waits_for_a_later_block(seed):
    rnd = random.Random(seed)
    nseq = rnd.randint(1, 4)
    lens_q = [rnd.choice([1, 77, 128, 300, 640, 1000, 2049]) for _ in range(nseq)]
    prior = [rnd.choice([0, 0, 129, 512, 700]) for _ in range(nseq)]
    lens_k = [q + p for q, p in zip(lens_q, prior)]
    causal = rnd.random() < 0.8
    window = rnd.choice([0, 0, 200, 513]) if causal else 0
    rep = rnd.choice([1, 2, 4])
    ctas = ctas_in_dispatch_order(lens_q, lens_k, causal, window, rep)
    for resident in (1, 2, 5):
        done, sem, order = replay(ctas, resident)
        assert done, (lens_q, lens_k, causal, window, rep, resident)
        touching = {}
        for _, _, its in ctas:
            for key, _, _ in its:
                touching[key] = touching.get(key, 0) + 1
        assert sem == touching
        for key, seq_of_tiles in order.items():
            assert seq_of_tiles == sorted(seq_of_tiles, reverse=True), (key, seq_of_tiles)


def test_ascending_dispatch_would_starve():
    """The same protocol with key tiles handed out in ascending order (the unordered kernel's mapping) cannot finish once
    the resident CTAs all wait for tiles that have not started: the reason the ordered mode reverses the mapping."""
    ctas = ctas_in_dispatch_order([2048], [2048], True, 0, 1, grid_slack=0)
    done, _, _ = replay(list(reversed(ctas)), resident=4)
    assert not done
