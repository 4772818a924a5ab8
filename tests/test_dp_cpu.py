"""Data-parallel host logic on CPU: gloo ranks for the collective path, and a single-process emulation of the
peer-memory kernels' shard arithmetic."""
import socket

import torch
import torch.multiprocessing as mp

import flextrain_b200 as ft
from flextrain_b200.parallel.comm import shard_range
from flextrain_b200.parallel.dp import build_segments, emulate_sharded_step
from conftest import build_tiny


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out):
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        am = build_tiny(world_size=world, rank=rank, batch_tokens=512)
        src = ft.SyntheticTokenSource(1024, 128, seed=7)
        losses = []
        for step in range(2):
            allseqs = src.get_sequences(512)
            mine = allseqs[rank::world]
            st = am.fwd_bwd(mine, loss_scale_factor=1.0 / 512, total_tokens_per_step=512)
            am.step()
            losses.append(st.loss_sum)
        flat = torch.cat([t.flatten().float() for _, _, _, t in am.named_master_params()])
        out.put((rank, losses, flat.numpy()))   # by value: a tensor would travel as a shared-memory handle that dies with the worker
    finally:
        dist.destroy_process_group()


def test_two_rank_collective_matches_single_process():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=300) for _ in range(world)], key=lambda x: x[0])
    res = [(r, l, torch.from_numpy(f)) for r, l, f in res]
    for p in procs:
        p.join(60)
    # single process on the union of the data
    am = build_tiny(batch_tokens=512)
    src = ft.SyntheticTokenSource(1024, 128, seed=7)
    tot = []
    for step in range(2):
        seqs = src.get_sequences(512)
        st = am.fwd_bwd(seqs, loss_scale_factor=1.0 / 512, total_tokens_per_step=512)
        am.step()
        tot.append(st.loss_sum)
    flat = torch.cat([t.flatten().float() for _, _, _, t in am.named_master_params()])
    for step in range(2):
        assert abs(res[0][1][step] + res[1][1][step] - tot[step]) < 1e-2
    for r in range(world):
        d = (res[r][2] - flat).abs()
        assert float(d.max()) < 2.5e-3 and float(d.mean()) < 2e-6
    assert torch.equal(res[0][2], res[1][2])


def test_shard_ranges_cover_exactly():
    for n in (1, 7, 8, 100, 4096, 1000003):
        for W in (1, 2, 3, 8):
            got, pos = 0, 0
            for r in range(W):
                b, c = shard_range(n, r, W)
                assert b == min(n, pos) or c == 0
                assert b % 8 == 0 or c == 0
                pos = b + c
                got += c
            assert got == n


def test_sharded_adamw_emulation_equals_plain_adamw():
    from flextrain_b200.ops import reference as ref
    am = build_tiny()
    bm = am.buffers
    lb = bm.layers[0]
    W = 4
    torch.manual_seed(1)
    pbuf = bm.param_buffer(0).clone()
    gbufs = []
    for r in range(W):
        g = torch.zeros_like(bm.grad_buffer(0))
        for name, (off, nb, shape, dt) in lb.g_layout.items():
            g[off:off + nb].view(dt).copy_(torch.randn(nb // 4) * 0.01)
        gbufs.append(g)
    segs_per_rank, states, total = [], [], 0
    for r in range(W):
        segs = build_segments(lb, 0, 0)
        off = 0
        for s in segs:
            s.begin, s.count = shard_range(s.numel, r, W)
            s.shard_off = off
            off += (s.count + 7) // 8 * 8
        segs_per_rank.append(segs)
        states.append((torch.zeros(off), torch.zeros(off)))
    pbufs = [pbuf.clone() for _ in range(W)]
    emulate_sharded_step(gbufs, pbufs, segs_per_rank, states, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, wd=0.1, step=1)
    # oracle: plain AdamW on the summed gradient
    want = pbuf.clone()
    gsum = sum(g.view(torch.float32) for g in gbufs)
    for t in lb.spec.trainable():
        off, nb, shape, dt = lb.p_layout[t.name]
        goff, gnb, _, gdt = lb.g_layout[t.grad_name]
        p = want[off:off + nb].view(dt)
        g = gsum[goff // 4:(goff + gnb) // 4]
        m, v = torch.zeros_like(p), torch.zeros_like(p)
        ref.adamw_step(p, g, m, v, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8,
                       weight_decay=0.0 if len(t.shape) == 1 else 0.1, step=1)
    for r in range(W):
        torch.testing.assert_close(pbufs[r].view(torch.float32), want.view(torch.float32), rtol=1e-5, atol=1e-7)


def test_p2p_takes_one_flag_epoch_per_fwd_bwd_call():
    """Host logic of the peer-memory path (no GPU): with two ``fwd_bwd`` calls before ``step()`` the reduce of the
    second call must wait on a NEW epoch; reusing the first call's epoch would let the wait pass at once while the
    peers are still accumulating.  Within one call all units share the epoch."""
    from types import SimpleNamespace
    from flextrain_b200.parallel.dp import P2PDataParallel

    class Group:
        def __init__(self): self.e = 0
        def next_epoch(self):
            self.e += 1
            return self.e

    dp = P2PDataParallel.__new__(P2PDataParallel)
    dp.group, dp._reduced_epoch = Group(), None
    dp.am = SimpleNamespace(step_num=0, fwd_bwd_serial=0)
    waited = []
    dp._reduce = lambda key: waited.append((key, dp._epoch))
    for call in (1, 2):                       # two calls of the same step
        dp.am.fwd_bwd_serial = call
        for layer in (1, 0):
            dp.on_layer_grads_ready(layer)
        dp.on_embed_head_grads_ready()
    dp.am.step_num, dp.am.fwd_bwd_serial = 1, 3   # next step
    dp.on_layer_grads_ready(1)
    assert [e for _, e in waited] == [1, 1, 1, 1, 2, 2, 2, 2, 3], waited
