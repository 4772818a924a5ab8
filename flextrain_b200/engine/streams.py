"""CUDA stream bundle and typed event maps (flextrain/engine/streams.py:46-277).

Waiting on an event that was never recorded raises ``KeyError`` instead of silently passing
(or hanging): a missing ``record`` is a scheduling bug and must fail loudly.  On CPU the bundle
degrades to no-op streams so the same engine code runs the parity configuration.
"""
from __future__ import annotations

import contextlib
import ctypes
from dataclasses import dataclass
from typing import Dict, Generic, Hashable, Optional, Tuple, TypeVar

import torch

K = TypeVar("K", bound=Hashable)


def _name_stream(stream, name: str) -> None:
    """Label a stream for profilers through NVTX (``nvtxNameCuStreamA``); best effort."""
    try:
        lib = ctypes.CDLL("libnvToolsExt.so.1")
        fn = lib.nvtxNameCuStreamA
        fn.argtypes = [ctypes.c_void_p, ctypes.c_char_p]
        fn.restype = None
        fn(ctypes.c_void_p(stream.cuda_stream), name.encode())
    except Exception:
        pass


class _NullStream:
    """Stand-in for a CUDA stream on CPU.  Every role gets its own instance so the protocol checker can tell the
    logical streams apart even though all work runs in program order."""

    def __init__(self, name: str = "null"):
        self.name = name

    def wait_stream(self, other): pass
    def wait_event(self, ev): pass
    def synchronize(self): pass
    def record_event(self, ev=None): return _NullEvent()


class _NullEvent:
    def record(self, stream=None): pass
    def wait(self, stream=None): pass
    def synchronize(self): pass
    def query(self): return True


@dataclass
class StreamBundle:
    compute: object
    inbound: object                    # host -> HBM (weights, grads, opt state, activations)
    outbound: object                   # HBM -> host
    inbound_fwd_context: object        # K/V / linear-state window refills
    comm: object                       # peer traffic (fused collectives)
    secondary_compute: Optional[object] = None
    is_cuda: bool = False
    checker: Optional[object] = None   # StreamProtocolChecker when FTB_STREAM_CHECK=1 / check=True

    ROLES = ("compute", "inbound", "outbound", "inbound_fwd_context", "comm")

    @classmethod
    def create(cls, device, secondary: bool = False, check: Optional[bool] = None) -> "StreamBundle":
        import os
        dev = torch.device(device)
        if dev.type != "cuda":
            b = cls(*[_NullStream(r) for r in cls.ROLES], _NullStream("secondary_compute") if secondary else None, False)
        else:
            with torch.cuda.device(dev):
                compute = torch.cuda.current_stream(dev)
                mk = lambda: torch.cuda.Stream(device=dev)
                b = cls(compute, mk(), mk(), mk(), mk(), mk() if secondary else None, True)
            for nm in ("inbound", "outbound", "inbound_fwd_context", "comm"):
                _name_stream(getattr(b, nm), "ftb." + nm)
        b._names = {id(getattr(b, r)): r for r in cls.ROLES}
        b._stack = []
        if check if check is not None else os.environ.get("FTB_STREAM_CHECK", "0") == "1":
            from .protocol_check import StreamProtocolChecker
            b.checker = StreamProtocolChecker()
        return b

    # ---- logical stream names (for the protocol checker)
    def name_of(self, stream) -> str:
        return self._names.get(id(stream), "other")

    def current(self) -> str:
        """Role of the stream that work issued now lands on (``use`` contexts nest; the default is compute)."""
        return self._stack[-1] if self._stack else "compute"

    @contextlib.contextmanager
    def use(self, stream):
        self._stack.append(self.name_of(stream))
        try:
            with (torch.cuda.stream(stream) if self.is_cuda else contextlib.nullcontext()):
                yield
        finally:
            self._stack.pop()

    def wait_stream(self, waiter, other) -> None:
        """``waiter`` waits for everything queued on ``other`` so far (logged for the protocol checker)."""
        waiter.wait_stream(other)
        if self.checker is not None:
            self.checker.wait_stream(self.name_of(waiter), self.name_of(other))

    def touch(self, resource, mode: str, note: str = "", stream=None) -> None:
        """Log a read (``"r"``) or write (``"w"``) of a tracked resource on ``stream`` (default: the current one)."""
        if self.checker is not None:
            self.checker.access(self.name_of(stream) if stream is not None else self.current(), resource, mode, note)

    def new_event(self):
        return torch.cuda.Event() if self.is_cuda else _NullEvent()

    def synchronize_all(self) -> None:
        for s in (self.compute, self.inbound, self.outbound, self.inbound_fwd_context, self.comm):
            s.synchronize()
        if self.checker is not None:
            self.checker.host_sync(self.ROLES)


class EventMap(Generic[K]):
    """``record(key, stream)`` / ``wait(key, stream)``; waiting on an unknown key raises ``KeyError``."""

    def __init__(self, bundle: StreamBundle, name: str):
        self.bundle, self.name = bundle, name
        self._ev: Dict[K, object] = {}

    def record(self, key: K, stream) -> None:
        ev = self.bundle.new_event()
        ev.record(stream) if self.bundle.is_cuda else None
        self._ev[key] = ev
        if self.bundle.checker is not None:
            self.bundle.checker.record((self.name, key), self.bundle.name_of(stream))

    def wait(self, key: K, stream) -> None:
        if key not in self._ev:
            raise KeyError(f"{self.name}: wait on never-recorded event {key!r}")
        if self.bundle.is_cuda:
            stream.wait_event(self._ev[key])
        if self.bundle.checker is not None:
            self.bundle.checker.wait((self.name, key), self.bundle.name_of(stream))

    def has(self, key: K) -> bool:
        return key in self._ev

    def pop(self, key: K) -> None:
        self._ev.pop(key, None)

    def clear(self) -> None:
        self._ev.clear()


LayerEventMap = EventMap[int]
SlotEventMap = EventMap[int]
LayerChunkEventMap = EventMap[Tuple[int, int]]


class EventBook:
    def __init__(self, bundle: StreamBundle):
        self.weights_in = LayerEventMap(bundle, "weights_in")
        self.grads_in = LayerEventMap(bundle, "grads_in")
        self.opt_in = LayerEventMap(bundle, "opt_in")
        self.layer_out = LayerEventMap(bundle, "layer_out")
        self.grads_ready = LayerEventMap(bundle, "grads_ready")
        self.act_out = LayerChunkEventMap(bundle, "act_out")
        self.act_in = LayerChunkEventMap(bundle, "act_in")
        self.act_computed = LayerChunkEventMap(bundle, "act_computed")
        self.slot_free = SlotEventMap(bundle, "slot_free")

    def clear_per_round(self) -> None:
        for m in (self.act_out, self.act_in, self.act_computed, self.slot_free):
            m.clear()
