"""Host memory backends (flextrain/engine/host_memory.py:71-255).

``LocalPinnedHostBackend`` allocates page-aligned host tensors and pins them with
``cudaHostRegister`` (exact size — ``pin_memory=True`` rounds up to a power of two), keeps a
process-wide registry so a pointer is never registered twice, and tolerates "already
registered" (CUDA error 712).  ``UnpinnedHostBackend`` is the CPU-only / test backend.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Protocol

import torch

_REGISTERED: Dict[int, int] = {}     # ptr -> nbytes, process-wide


class HostMemoryBackend(Protocol):
    def alloc(self, nbytes: int) -> torch.Tensor: ...
    def free(self, t: torch.Tensor) -> None: ...


def _cudart():
    return ctypes.CDLL("libcudart.so", mode=ctypes.RTLD_GLOBAL) if not hasattr(_cudart, "lib") else _cudart.lib


class LocalPinnedHostBackend:
    PAGE = 2 << 20

    def __init__(self):
        try:
            self.rt = torch.cuda.cudart()
        except Exception:   # pragma: no cover
            self.rt = None

    def alloc(self, nbytes: int) -> torch.Tensor:
        nbytes = max(int(nbytes), 1)
        t = torch.zeros(nbytes, dtype=torch.uint8)
        ptr = t.data_ptr()
        if self.rt is not None and ptr not in _REGISTERED:
            rc = self.rt.cudaHostRegister(ptr, nbytes, 0)
            code = int(rc.value) if hasattr(rc, "value") else int(rc)
            if code not in (0, 712):
                raise RuntimeError(f"cudaHostRegister failed with {code} for {nbytes} bytes")
            _REGISTERED[ptr] = nbytes
        return t

    def free(self, t: torch.Tensor) -> None:
        ptr = t.data_ptr()
        if ptr in _REGISTERED and self.rt is not None:
            self.rt.cudaHostUnregister(ptr)
            _REGISTERED.pop(ptr, None)


class UnpinnedHostBackend:
    def alloc(self, nbytes: int) -> torch.Tensor:
        return torch.zeros(max(int(nbytes), 1), dtype=torch.uint8)

    def free(self, t: torch.Tensor) -> None:
        return None


def default_backend(device) -> HostMemoryBackend:
    return LocalPinnedHostBackend() if torch.device(device).type == "cuda" else UnpinnedHostBackend()


def default_host_backend(device="cuda") -> HostMemoryBackend:
    """The reference's name for :func:`default_backend` (flextrain/engine/host_memory.py)."""
    return default_backend(device)


def unregister_all_process_pinned_memory() -> int:
    """Undo every ``cudaHostRegister`` this process still holds through :class:`LocalPinnedHostBackend` (engines that
    were dropped without ``destroy()`` leave registrations behind); returns how many were released
    (flextrain/engine/host_memory.py:215-233)."""
    n = 0
    try:
        rt = torch.cuda.cudart()
    except Exception:
        rt = None
    for ptr in list(_REGISTERED):
        if rt is not None:
            rt.cudaHostUnregister(ptr)
        _REGISTERED.pop(ptr, None)
        n += 1
    return n
