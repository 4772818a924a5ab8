"""Python face of the C++ copy engine (``csrc/copy_engine.cpp``).

``CopyEngine.submit`` takes a list of transfers ``(dst, src, stream, wait_key, wait_event, record_key)`` and
returns immediately; ``stream_wait(key, ticket, stream)`` makes a CUDA stream wait for a recorded transfer.
On CPU the engine runs in host-only mode (plain memcpy in the worker thread) so the same scheduling code is
exercised by the CPU tests.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_uint64, c_void_p
from typing import Sequence, Tuple

import torch

INBOUND, OUTBOUND, CONTEXT = 0, 1, 2


class CopyEngine:
    def __init__(self, device):
        from ..ops.cuda import load
        self.lib = load("copy_engine")
        self.lib.ftb_ce_create.restype = c_void_p
        self.lib.ftb_ce_submit.restype = c_uint64
        dev = torch.device(device)
        self.device = dev
        idx = (dev.index if dev.index is not None else torch.cuda.current_device()) if dev.type == "cuda" else -1
        self.h = c_void_p(self.lib.ftb_ce_create(c_int(idx)))
        if not self.h:
            raise RuntimeError("copy engine could not create its streams")
        self._keep = []

    def submit(self, jobs: Sequence[Tuple]) -> int:
        """``jobs``: ``(dst_tensor, src_tensor, stream, wait_key, wait_event, record_key)``; returns a ticket."""
        n = len(jobs)
        if n == 0:
            return 0
        dst = (c_void_p * n)(*[j[0].data_ptr() for j in jobs])
        src = (c_void_p * n)(*[j[1].data_ptr() for j in jobs])
        for j in jobs:
            assert j[0].numel() * j[0].element_size() == j[1].numel() * j[1].element_size(), "size mismatch"
        nb = (c_uint64 * n)(*[j[0].numel() * j[0].element_size() for j in jobs])
        st = (c_int * n)(*[j[2] for j in jobs])
        wk = (c_uint64 * n)(*[j[3] or 0 for j in jobs])
        we = (c_void_p * n)(*[(j[4].cuda_event if j[4] is not None else 0) for j in jobs])
        rk = (c_uint64 * n)(*[j[5] or 0 for j in jobs])
        self._keep = [j[4] for j in jobs if j[4] is not None][-64:] + self._keep[-64:]
        return int(self.lib.ftb_ce_submit(self.h, c_int(n), dst, src, nb, st, wk, we, rk))

    def stream_wait(self, key: int, ticket: int, stream=None) -> None:
        s = stream.cuda_stream if stream is not None and hasattr(stream, "cuda_stream") else 0
        rc = self.lib.ftb_ce_stream_wait(self.h, c_uint64(key), c_uint64(ticket), c_void_p(s))
        if rc == -5:
            raise KeyError(f"copy engine: wait on never-recorded event {key}")
        if rc != 0:
            raise RuntimeError(f"copy engine stream_wait failed ({rc})")

    def flush(self, ticket: int) -> None:
        rc = self.lib.ftb_ce_flush(self.h, c_uint64(ticket))
        if rc != 0:
            raise RuntimeError(f"copy engine error {rc}")

    def synchronize(self) -> None:
        rc = self.lib.ftb_ce_synchronize(self.h)
        if rc != 0:
            raise RuntimeError(f"copy engine error {rc}")

    def stats(self) -> Tuple[int, int]:
        b, c = c_uint64(), c_uint64()
        self.lib.ftb_ce_stats(self.h, ctypes.byref(b), ctypes.byref(c))
        return int(b.value), int(c.value)

    def close(self) -> None:
        if self.h:
            self.lib.ftb_ce_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
