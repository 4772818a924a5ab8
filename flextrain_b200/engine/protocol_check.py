"""Host-side stream-protocol checker: a vector-clock race detector over the engine's streams.

The engine moves ring slots (weights, gradients, optimizer state), the host activation arena and the K/V window
between streams with events.  A missing ``wait`` does not crash: it silently trains on stale or half-written bytes.
``compute-sanitizer`` would find some of these on a GPU; this checker finds the ordering bug itself, on the host,
on CPU or GPU, by replaying the happens-before graph the engine builds:

* every stream carries a vector clock; an operation on a stream ticks its own component;
* ``record(event, stream)`` snapshots the stream's clock, ``wait(event, stream)`` joins that snapshot into the
  waiting stream, ``wait_stream(a, b)`` joins b's clock into a, a host synchronisation joins everything;
* every access to a tracked resource (``("p", slot)``, ``("g", slot)``, ``("o", slot)``, a host arena range, the K/V
  window) is logged with the accessing stream's clock.  A write must happen-after every earlier read and write of the
  resource, a read after the last write; anything else is a violation, recorded with both access sites.

Enable with ``FTB_STREAM_CHECK=1`` (or ``StreamBundle.create(..., check=True)``); ``ActiveModel.protocol_violations()``
returns what was found.  The reference keeps this safety by construction only — typed event maps and comments that pin
which stream a copy must be issued on (flextrain/engine/streams.py:186-202, flextrain/engine/active_model.py:579-585).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Tuple

Clock = Dict[str, int]


def _join(dst: Clock, src: Clock) -> None:
    for k, v in src.items():
        if dst.get(k, 0) < v:
            dst[k] = v


def _happens_before(snap: Clock, now: Clock) -> bool:
    return all(now.get(k, 0) >= v for k, v in snap.items())


@dataclass
class Violation:
    resource: Hashable
    kind: str                 # "write-after-read", "write-after-write", "read-after-write"
    stream: str
    note: str
    earlier_stream: str
    earlier_note: str

    def __str__(self) -> str:
        return (f"{self.kind} on {self.resource!r}: {self.stream} ({self.note}) is not ordered after "
                f"{self.earlier_stream} ({self.earlier_note})")


@dataclass
class _History:
    write: Optional[Tuple[Clock, str, str]] = None                       # (clock, stream, note)
    reads: List[Tuple[Clock, str, str]] = field(default_factory=list)


class StreamProtocolChecker:
    def __init__(self):
        self.clocks: Dict[str, Clock] = {}
        self.events: Dict[Hashable, Clock] = {}
        self.history: Dict[Hashable, _History] = {}
        self.violations: List[Violation] = []
        self.n_accesses = 0

    # ------------------------------------------------------------------ clocks
    def _clock(self, stream: str) -> Clock:
        return self.clocks.setdefault(stream, {stream: 0})

    def _tick(self, stream: str) -> Clock:
        c = self._clock(stream)
        c[stream] = c.get(stream, 0) + 1
        return c

    def record(self, event: Hashable, stream: str) -> None:
        self.events[event] = dict(self._tick(stream))

    def wait(self, event: Hashable, stream: str) -> None:
        snap = self.events.get(event)
        if snap is not None:
            _join(self._clock(stream), snap)

    def wait_stream(self, waiter: str, other: str) -> None:
        _join(self._clock(waiter), self._tick(other))

    def host_sync(self, streams) -> None:
        """The host waited for every stream: everything issued so far happens-before everything issued later."""
        top: Clock = {}
        for s in streams:
            _join(top, self._tick(s))
        for s in streams:
            _join(self._clock(s), top)

    # ---------------------------------------------------------------- accesses
    def access(self, stream: str, resource: Hashable, mode: str, note: str = "") -> None:
        now = dict(self._tick(stream))
        h = self.history.setdefault(resource, _History())
        self.n_accesses += 1
        if h.write is not None and not _happens_before(h.write[0], now):
            self.violations.append(Violation(resource, "write-after-write" if mode == "w" else "read-after-write",
                                             stream, note, h.write[1], h.write[2]))
        if mode == "w":
            for snap, s2, n2 in h.reads:
                if not _happens_before(snap, now):
                    self.violations.append(Violation(resource, "write-after-read", stream, note, s2, n2))
            h.write, h.reads = (now, stream, note), []
        else:
            h.reads.append((now, stream, note))

    def forget(self, prefix: Hashable) -> None:
        """Drop the history of resources whose key starts with ``prefix`` (a re-allocated arena)."""
        for k in [k for k in self.history if isinstance(k, tuple) and k[:1] == (prefix,)]:
            del self.history[k]
