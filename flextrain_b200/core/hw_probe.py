"""Hardware probe (flextrain/core/hw_probe.py:71-328): sustained bf16 GEMM rate, HBM bandwidth, PCIe bandwidth.

* GEMM: 8192^3 bf16 on this package's tcgen05 kernel for ``seconds`` in two halves; the second half wins, which
  excludes the boost clocks a 1 kW part cannot hold (the reference uses 4096^3 for 7 s the same way).
* HBM: a large device-to-device copy (read + write bytes).
* PCIe: concurrent pinned H2D and D2H copies of 256 MiB on two streams.
* NVLink: left at the measured peer-copy figure unless a peer buffer is supplied.
"""
from __future__ import annotations

import time

import torch

from .save_level import HardwareCost


def _timed(fn, seconds: float):
    torch.cuda.synchronize()
    n, t0 = 0, time.perf_counter()
    while True:
        for _ in range(4):
            fn()
        n += 4
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if dt >= seconds:
            return n, dt


def probe_matmul(device, seconds: float = 4.0, n: int = 8192) -> float:
    from .. import ops
    a = torch.randn(n, n, device=device, dtype=torch.bfloat16)
    b = torch.randn(n, n, device=device, dtype=torch.bfloat16)
    out = torch.empty(n, n, device=device, dtype=torch.bfloat16)
    fn = lambda: ops.gemm(a, b, trans_b=True, out=out)
    _timed(fn, seconds / 2)
    cnt, dt = _timed(fn, seconds / 2)
    return 2.0 * n ** 3 * cnt / dt / 1e12


def probe_hbm(device, seconds: float = 1.0, nbytes: int = 2 << 30) -> float:
    a = torch.empty(nbytes, dtype=torch.uint8, device=device)
    b = torch.empty_like(a)
    cnt, dt = _timed(lambda: b.copy_(a), seconds)
    return 2.0 * nbytes * cnt / dt / 1e9


def probe_pcie(device, seconds: float = 1.0, nbytes: int = 256 << 20) -> float:
    h1 = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    h2 = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d1 = torch.empty(nbytes, dtype=torch.uint8, device=device)
    d2 = torch.empty(nbytes, dtype=torch.uint8, device=device)
    s1, s2 = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)

    def both():
        with torch.cuda.stream(s1):
            d1.copy_(h1, non_blocking=True)
        with torch.cuda.stream(s2):
            h2.copy_(d2, non_blocking=True)

    cnt, dt = _timed(both, seconds)
    return nbytes * cnt / dt / 1e9       # per direction, with both directions busy


def probe_hardware(device="cuda:0", seconds: float = 6.0, verbose: bool = False) -> HardwareCost:
    dev = torch.device(device)
    if dev.type != "cuda":
        return HardwareCost()
    with torch.cuda.device(dev):
        tf = probe_matmul(dev, seconds * 0.6)
        hbm = probe_hbm(dev, seconds * 0.2)
        pcie = probe_pcie(dev, seconds * 0.2)
    if verbose:
        print(f"[hw probe] bf16 {tf:.0f} TFLOPS sustained, HBM {hbm:.0f} GB/s, PCIe {pcie:.1f} GB/s per direction")
    return HardwareCost(peak_tflops=tf, pcie_bw_gbps=pcie, mem_bw_gbps=hbm)
