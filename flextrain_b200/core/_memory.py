"""Memory discovery (flextrain/core/_memory.py:33-307).

GPU: ``torch.cuda.mem_get_info`` → ``nvidia-smi`` fallback.  Host: the tightest of Slurm's allocation
(``SLURM_MEM_PER_NODE`` / ``SLURM_MEM_PER_CPU``), the cgroup v2 / v1 limit minus current usage, and the
kernel's MemAvailable (psutil when present); this process's own RSS is added back since it is already
part of the budget it is about to fill.
"""
from __future__ import annotations

import os
import subprocess
from typing import Optional


def get_available_gpu_memory(device="cuda:0", *, device_id: Optional[int] = None) -> int:
    """Free device memory in bytes; ``device`` is a device string / object or a bare index (``device_id`` is the
    reference's keyword for the index)."""
    import torch
    if device_id is not None:
        device = device_id
    dev = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
    if dev.type != "cuda":
        return 8 << 30
    try:
        free, _ = torch.cuda.mem_get_info(dev)
        return int(free)
    except Exception:
        pass
    try:
        out = subprocess.run(["nvidia-smi", "--query-gpu=memory.free", "--format=csv,noheader,nounits", "-i",
                              str(dev.index or 0)], capture_output=True, text=True, timeout=10).stdout
        return int(float(out.strip().splitlines()[0])) << 20
    except Exception:
        return 0


def _read_int(path: str) -> Optional[int]:
    try:
        with open(path) as f:
            s = f.read().strip()
        return None if s in ("max", "") else int(s)
    except (OSError, ValueError):
        return None


def _cgroup_available() -> Optional[int]:
    lim, use = _read_int("/sys/fs/cgroup/memory.max"), _read_int("/sys/fs/cgroup/memory.current")
    if lim is None:
        lim = _read_int("/sys/fs/cgroup/memory/memory.limit_in_bytes")
        use = _read_int("/sys/fs/cgroup/memory/memory.usage_in_bytes")
    if lim is None or lim > (1 << 60):
        return None
    return max(0, lim - (use or 0))


def _slurm_limit() -> Optional[int]:
    if "SLURM_MEM_PER_NODE" in os.environ:
        return int(os.environ["SLURM_MEM_PER_NODE"]) << 20
    if "SLURM_MEM_PER_CPU" in os.environ:
        cpus = int(os.environ.get("SLURM_CPUS_ON_NODE", os.environ.get("SLURM_CPUS_PER_TASK", "1")))
        return (int(os.environ["SLURM_MEM_PER_CPU"]) * cpus) << 20
    return None


def _meminfo_available() -> Optional[int]:
    try:
        import psutil
        return int(psutil.virtual_memory().available)
    except Exception:
        pass
    try:
        with open("/proc/meminfo") as f:
            for line in f:
                if line.startswith("MemAvailable:"):
                    return int(line.split()[1]) << 10
    except OSError:
        pass
    return None


def _own_rss() -> int:
    try:
        import psutil
        p = psutil.Process()
        return int(p.memory_info().rss + sum(c.memory_info().rss for c in p.children(recursive=True)))
    except Exception:
        return 0


def get_available_host_memory() -> int:
    cands = [x for x in (_slurm_limit(), _cgroup_available(), _meminfo_available()) if x is not None]
    if not cands:
        return 16 << 30
    return int(min(cands) + _own_rss())
