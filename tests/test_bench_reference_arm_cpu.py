"""The reference arm's plan ladder, walked on two CPU ranks against a stand-in ``flextrain`` package.

What is pinned here is the control flow only: the ranks stay in lock-step when a plan is refused, when one rank's
engine raises in forward / backward or in the optimizer step, and when a later warm-up step fails; every engine that
was built is given back before the next one is planned; the gradient sum runs on every rank of every completed step;
and exactly one JSON line comes out.  The stand-in engine fails where an environment variable tells it to.
"""
import json
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

FAKE = {
    "flextrain/__init__.py": '''
        import json, os
        import torch
        import torch.distributed as dist
        LOG = os.environ["FAKE_REF_LOG"]
        PLAN = json.loads(os.environ["FAKE_REF_PLAN"])          # {"<gpu gib or none>": behaviour}
        LIVE = []                                                # engines that were built and not yet given back

        def _rank():
            return dist.get_rank() if dist.is_initialized() else 0

        def _world():
            return dist.get_world_size() if dist.is_initialized() else 1

        def _log(what):
            with open(LOG + f".{_rank()}", "a") as f:
                f.write(what + "\\n")

        class _Stats:
            def __init__(self, loss): self.total_loss = loss

        class _WS:
            target_round_tokens, max_chunk_size, n_gpu_layers, n_gpu_grads, n_gpu_opt_layers = 4096, 2048, 3, 2, 1
            host_act_buffer_size = 1 << 30

        class _Buffers:
            def __init__(self):
                self.host_grads = [{"w": torch.zeros(4)}, {"w": torch.zeros(4)}]
                self.gpu_embed_grads = {"e": torch.zeros(2)}
                self.destroyed = False
            def destroy(self):
                self.destroyed = True

        class _Engine:
            def __init__(self, key, how):
                self.key, self.how, self.buffers, self.working_set, self.n = key, how, _Buffers(), _WS(), 0
                LIVE.append(self)
            def _maybe(self, where):
                for rule in self.how.get("raise", []):          # {"where": "fwd_bwd"|"step", "rank": r, "call": n}
                    if rule["where"] == where and rule["rank"] == _rank() and rule["call"] == self.n:
                        raise RuntimeError(f"CUDA out of memory (stand-in) in {where} call {self.n}")
            def fwd_bwd(self, seqs, loss_scale_factor, total_tokens_per_step):
                self.n += 1
                assert len(LIVE) == 1 and LIVE[0] is self, "an earlier engine was not given back"
                self._maybe("fwd_bwd")
                for d in self.buffers.host_grads:
                    d["w"].fill_(float(_rank() + 1))
                self.buffers.gpu_embed_grads["e"].fill_(float(_rank() + 1))
                return _Stats(12.5 * sum(len(s.tokens) for s in seqs))
            def step(self):
                want = float(sum(r + 1 for r in range(_world())))
                for d in self.buffers.host_grads:               # the ranks' gradients were summed before the update
                    assert bool((d["w"] == want).all()), (d["w"], want)
                assert bool((self.buffers.gpu_embed_grads["e"] == want).all())
                self._maybe("step")
                _log(f"step {self.key} {self.n}")

        def from_dims(dims, arch, optimizer, max_seq_len, max_global_batch_tokens, max_gpu_mem_bytes,
                      max_host_mem_bytes, max_chunk_size=None, hw_cost=None, mem_bw_gbps=None, hyperparams=None,
                      device=None, verbose=False):
            gib = max_gpu_mem_bytes >> 30
            key = "none" if gib >= 170 else str(gib)
            how = PLAN.get(key + "/" + str(max_chunk_size), PLAN.get(key, {}))
            _log(f"from_dims {key} chunk={max_chunk_size} state={optimizer.state_dtype}")
            if how.get("refuse"):
                raise ValueError("GPU memory capacity bound (stand-in)")
            if how.get("build_oom_rank") == _rank():
                raise RuntimeError("cudaHostRegister failed (stand-in)")
            return _Engine(key, how)
    ''',
    "flextrain/core/__init__.py": "",
    "flextrain/core/_memory.py": "def get_available_host_memory():\n    return 64 << 30\n",
    "flextrain/core/save_level.py": '''
        from dataclasses import dataclass
        @dataclass
        class HardwareCost:
            peak_tflops: float
            pcie_bw_gbps: float
    ''',
    "flextrain/core/hw_probe.py": '''
        from .save_level import HardwareCost
        class _Probe:
            hw_cost, mem_bw_gbps = HardwareCost(1400.0, 40.0), 6500.0
        def probe_hardware(device=None):
            return _Probe()
    ''',
    "flextrain/io/__init__.py": "",
    "flextrain/io/sequence.py": "class Sequence:\n    def __init__(self, tokens):\n        self.tokens = tokens\n",
    "flextrain/io/sources.py": '''
        from .sequence import Sequence
        class SyntheticTokenSource:
            def __init__(self, vocab, seq_len, seed=0):
                self.seq_len = seq_len
            def get_sequences(self, n_tokens):
                return [Sequence([0] * self.seq_len) for _ in range(n_tokens // self.seq_len)]
    ''',
    "flextrain/optim/__init__.py": "",
    "flextrain/optim/adamw.py": '''
        class AdamWHyperparams:
            def __init__(self, **kw): self.__dict__.update(kw)
        class AdamW:
            def __init__(self, hp, state_dtype=None): self.hp, self.state_dtype = hp, state_dtype
    ''',
    "flextrain/engine/__init__.py": '''
        def unregister_all_process_pinned_memory():
            import flextrain
            for e in list(flextrain.LIVE):
                if e.buffers.destroyed:
                    flextrain.LIVE.remove(e)
            flextrain._log("unregister_all")
    ''',
}

DRIVER = '''
import os, sys, time
sys.path.insert(0, {root!r})
import torch, torch.distributed as dist
import bench

bench.ROOT = {fake_root!r}
bench._device_of = lambda local: "cpu"
torch.cuda.set_device = lambda d: None
torch.cuda.mem_get_info = lambda *a: (178 << 30, 180 << 30)
torch.cuda.synchronize = lambda *a: None
torch.cuda.empty_cache = lambda: None

class _Event:
    def __init__(self, enable_timing=False): self.t = None
    def record(self, *a): self.t = time.perf_counter()
    def elapsed_time(self, other): return (other.t - self.t) * 1e3 + 1.0
torch.cuda.Event = _Event

_init = dist.init_process_group
dist.init_process_group = lambda backend, **kw: _init("gloo")
sys.argv = ["bench.py", "--impl", "reference", "--small", "--steps", "2", "--warmup", "2", "--gpus", {world!r}]
bench.main()
'''


def _run(tmp_path, plan: dict, world: int):
    fake_root = tmp_path / "root"
    for rel, body in FAKE.items():
        f = fake_root / "baseline" / "_ref" / rel
        f.parent.mkdir(parents=True, exist_ok=True)
        f.write_text(textwrap.dedent(body))
    drv = tmp_path / "drive.py"
    drv.write_text(DRIVER.format(root=ROOT, fake_root=str(fake_root), world=str(world)))
    log = str(tmp_path / "log")
    env = dict(os.environ, FAKE_REF_LOG=log, FAKE_REF_PLAN=json.dumps(plan), CUDA_VISIBLE_DEVICES="")
    if world == 1:
        cmd = [sys.executable, str(drv)]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", "29631", str(drv)]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=str(tmp_path))
    logs = [open(f"{log}.{r}").read().splitlines() if os.path.exists(f"{log}.{r}") else [] for r in range(world)]
    return p, logs


def _json_line(p):
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, (p.stdout, p.stderr[-3000:])
    return json.loads(lines[0])


def test_first_plan_that_survives_its_warmup_runs_on_two_ranks(tmp_path):
    """Whole-GPU plan: rank 1 runs out of memory in its first forward / backward.  150 GiB: refused by the planner
    without a chunk cap and with the probed link figures, built with the cap, then rank 0 fails in the optimizer step
    of the second warm-up step.  120 GiB: rank 1 cannot pin its host memory.  96 GiB runs."""
    plan = {"none": {"raise": [{"where": "fwd_bwd", "rank": 1, "call": 1}]},
            "150/None": {"refuse": True},
            "150/16384": {"raise": [{"where": "step", "rank": 0, "call": 2}]},
            "120": {"build_oom_rank": 1},
            "96": {}}
    p, logs = _run(tmp_path, plan, world=2)
    assert p.returncode == 0, p.stderr[-3000:]
    obj = _json_line(p)
    assert obj["impl"] == "reference" and "unavailable" not in obj, obj
    assert obj["n_gpus"] == 2 and obj["steps"] == 2 and obj["value"] > 0
    assert obj["config"]["plan"] == {"opt_state": "float32", "hw_cost": "probed", "max_gpu_gib": 96, "max_chunk_size": None}
    assert abs(obj["loss_step1"] - 12.5) < 1e-9 and abs(obj["loss"] - 12.5) < 1e-9      # job mean over both ranks' halves
    for r in (0, 1):
        builds = [l for l in logs[r] if l.startswith("from_dims")]
        # both ranks planned the same sequence of rungs: the failed whole-GPU plan is not retried with other link /
        # chunk variants, the refused 150 GiB plan is (nominal link first would come after every chunk cap)
        assert [b.split()[1] + "/" + b.split()[2] for b in builds if "verbose" not in b][:2] == ["none/chunk=None", "150/chunk=None"]
        assert builds[-1].startswith("from_dims 96 chunk=None")
        steps = [l for l in logs[r] if l.startswith("step")]
        # 150 GiB: one complete step (the second failed on rank 0 before / after its update); 96 GiB: 2 warm-up + 2 timed
        assert [s for s in steps if s.startswith("step 96")] == [f"step 96 {i}" for i in (1, 2, 3, 4)]
        assert not any(s.startswith("step none") for s in steps)
    assert "attempt failed" in p.stderr and "warm-up step 2" in p.stderr


def test_no_plan_runs_gives_the_unavailable_line(tmp_path):
    plan = {k: {"refuse": True} for k in ("none", "150", "120", "96", "64", "31")}
    p, _ = _run(tmp_path, plan, world=1)
    assert p.returncode == 0, p.stderr[-3000:]
    obj = _json_line(p)
    assert obj["impl"] == "reference" and "no plan builds" in obj["unavailable"]


def test_a_failed_timed_step_ends_every_rank_with_the_unavailable_line(tmp_path):
    """Warm-up passes, then rank 1's engine raises in the first timed step: both ranks leave together (no rank waits
    in the gradient all-reduce) and rank 0 prints the ``unavailable`` line."""
    plan = {"none": {"raise": [{"where": "fwd_bwd", "rank": 1, "call": 3}]}}
    p, logs = _run(tmp_path, plan, world=2)
    assert p.returncode == 0, p.stderr[-3000:]
    obj = _json_line(p)
    assert "a timed step failed" in obj["unavailable"]
    assert [l for l in logs[0] if l.startswith("step")] == ["step none 1", "step none 2"]
