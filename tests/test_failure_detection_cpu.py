"""Failure detection on the host (no GPU, nothing faults): ranks as CPU processes around a TCPStore / gloo group.

* a rank that leaves between steps is announced through the heartbeat and raises ``PeerLost`` on the survivor;
* a rank that goes silent is detected after the staleness limit;
* a rank that dies before joining a collective makes the survivor's collective fail with an error (bounded by the
  process-group timeout) instead of hanging."""
import datetime
import os
import socket
import time

import pytest
import torch
import torch.multiprocessing as mp

from flextrain_b200.parallel.health import Heartbeat, PeerLost


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _hb_worker(rank, port, mode, out):
    import torch.distributed as dist
    store = dist.TCPStore("127.0.0.1", port, 2, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    hb = Heartbeat(store, rank, 2, stale_s=1.0, max_lag=2)
    try:
        if rank == 1:
            for step in range(3):
                hb.beat(step)
                time.sleep(0.05)
            if mode == "leave":
                hb.leave("finished early")
            else:                       # go silent but stay alive for a while
                time.sleep(4.0)
            out.put((rank, "done"))
            return
        result = "no failure seen"
        for step in range(200):
            hb.beat(step % 3)           # stay within max_lag of the peer: only departure / silence may trigger
            try:
                hb.check(grace_s=5.0)
            except PeerLost as e:
                result = f"lost:{e.rank}:{e.why}"
                break
            time.sleep(0.05)
        out.put((rank, result))
        time.sleep(0.5)                 # keep the store's master alive until the peer has finished
    except Exception as e:              # pragma: no cover
        out.put((rank, f"error:{type(e).__name__}:{e}"))


@pytest.mark.parametrize("mode", ["leave", "silent"])
def test_heartbeat_reports_lost_peer(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_hb_worker, args=(r, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=60) for _ in range(2))
    for p in procs:
        p.join(30)
    assert res[1] == "done"
    assert res[0].startswith("lost:1:"), res
    if mode == "leave":
        assert "finished early" in res[0]
    else:
        assert "no heartbeat" in res[0]


def test_heartbeat_lag_and_missing_peer():
    class DictStore:                     # the subset of the store interface the heartbeat uses
        def __init__(self): self.d = {}
        def set(self, k, v): self.d[k] = v.encode()
        def get(self, k): return self.d[k]
        def check(self, ks): return all(k in self.d for k in ks)
    st = DictStore()
    a, b = Heartbeat(st, 0, 2, max_lag=1), Heartbeat(st, 1, 2, max_lag=1)
    a.beat(0)
    with pytest.raises(PeerLost, match="never reported"):
        a.check()
    a.check(grace_s=1.0)                 # start-up skew tolerated
    b.beat(0); a.beat(1); a.check()
    a.beat(3)
    with pytest.raises(PeerLost, match="steps behind"):
        a.check()


def _collective_worker(rank, port, out):
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=2,
                            timeout=datetime.timedelta(seconds=8))
    t = torch.ones(4)
    dist.all_reduce(t)                   # both ranks take part in the first one
    if rank == 1:
        os._exit(0)                      # dies between steps, without announcing it
    t0 = time.time()
    try:
        dist.all_reduce(t)
        out.put("second collective returned")
    except Exception as e:
        out.put(f"raised:{type(e).__name__}:{time.time() - t0:.1f}")


def test_collective_with_dead_peer_raises_instead_of_hanging():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_collective_worker, args=(r, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    msg = q.get(timeout=90)
    for p in procs:
        p.join(30)
    assert msg.startswith("raised:"), msg
    assert float(msg.rsplit(":", 1)[1]) < 30.0


def test_training_loop_stops_on_a_device_status_word(tmp_path, monkeypatch):
    """A bounded device-side wait that runs out leaves an error word and lets the step finish on incomplete data.
    ``ActiveModel.check_health`` turns a non-zero word into an exception, and ``train.py`` calls it after every
    step: with a fake status injected at step 2 the loop must stop there instead of training on."""
    import importlib.util
    import sys
    from flextrain_b200.engine.active_model import ActiveModel

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    spec = importlib.util.spec_from_file_location("ftb_train_cli", os.path.join(root, "train.py"))
    train = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(train)

    real = ActiveModel.check_health
    calls = []

    def fake(self, error_words=None):
        calls.append(self.step_num)
        # step 2: the word a run-out wait for peer panel 1 would leave in the GEMM library
        return real(self, error_words={"gemm_tcgen05": 2041} if self.step_num == 2 else {})

    monkeypatch.setattr(ActiveModel, "check_health", fake)
    monkeypatch.chdir(tmp_path)
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "")
    argv = ["--model", "dims:tiny_llama", "--mode", "full", "--data-source", "synthetic", "--max-seq-len", "128",
            "--max-global-batch-tokens", "512", "--steps", "4", "--lr", "1e-3", "--output-dir", str(tmp_path / "o")]
    with pytest.raises(RuntimeError, match="device-side wait or check failed during step 2.*2041"):
        train.main(argv)
    assert calls == [1, 2]


def test_check_health_passes_on_clean_words_and_polls_groups():
    from flextrain_b200.engine.active_model import ActiveModel

    class Grp:
        def __init__(self): self.n = 0
        def check(self): self.n += 1

    class Streams:
        def synchronize_all(self): pass

    am = ActiveModel.__new__(ActiveModel)
    am.streams, am.device, am.step_num = Streams(), torch.device("cpu"), 7
    am.dp, am.ep, am.tp = Grp(), None, Grp()
    am.check_health(error_words={"comm": 0, "moe": 0})
    assert am.dp.n == 1 and am.tp.n == 1
    with pytest.raises(RuntimeError, match="step 7"):
        am.check_health(error_words={"comm": 1003})
