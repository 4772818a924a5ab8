"""Host-side failure detection between the ranks of one job.

The peer-memory kernels never wait without a limit (a missing peer ends a wait with an error status that
``PeerGroup.check`` raises on the host), but a limit of seconds is a long time to find out that a peer is gone.  The
heartbeat makes the ranks learn of it on the host, between steps and before the next launch: every rank writes
``(step, wall time)`` into the job's key-value store when it finishes a step and, before it starts the next one, reads
its peers' entries.  A peer that announced its departure (``leave``), stopped beating for longer than ``stale_s``, or
fell more than ``max_lag`` steps behind raises :class:`PeerLost` on everyone else — with no kernel or collective in
flight, so the survivors' CUDA contexts stay usable (save a checkpoint, shrink the job, exit cleanly).

The reference project is single-process and has no failure detection (nothing to cite); the store is any
``torch.distributed`` store (``TCPStore``, ``FileStore``, or the default process group's store).
"""
from __future__ import annotations

import time
from typing import List, Optional


class PeerLost(RuntimeError):
    def __init__(self, rank: int, why: str):
        super().__init__(f"rank {rank} is gone: {why}")
        self.rank, self.why = rank, why


class Heartbeat:
    def __init__(self, store, rank: int, world: int, *, prefix: str = "ftb_hb", stale_s: float = 60.0,
                 max_lag: int = 2):
        self.store, self.rank, self.world = store, rank, world
        self.prefix, self.stale_s, self.max_lag = prefix, stale_s, max_lag
        self.step = -1

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        """Call when a step has finished (nothing of this rank is in flight any more)."""
        self.step = step
        self.store.set(self._key(self.rank), f"{step}:{time.time():.3f}")

    def leave(self, reason: str = "left") -> None:
        """Announce an orderly departure; call between steps, then exit."""
        self.store.set(self._key(self.rank), f"gone:{reason}")

    def peers(self) -> List[Optional[str]]:
        out: List[Optional[str]] = []
        for r in range(self.world):
            k = self._key(r)
            out.append(self.store.get(k).decode() if self.store.check([k]) else None)
        return out

    def check(self, grace_s: float = 0.0) -> None:
        """Raise :class:`PeerLost` if a peer left, went silent, or lags.  ``grace_s``: how long a peer may still be
        missing its FIRST beat (start-up skew)."""
        now = time.time()
        for r, v in enumerate(self.peers()):
            if r == self.rank:
                continue
            if v is None:
                if grace_s <= 0:
                    raise PeerLost(r, "never reported")
                continue
            if v.startswith("gone:"):
                raise PeerLost(r, v[5:])
            step_s, ts_s = v.split(":")
            if now - float(ts_s) > self.stale_s:
                raise PeerLost(r, f"no heartbeat for {now - float(ts_s):.1f}s (limit {self.stale_s}s)")
            if self.step - int(step_s) > self.max_lag:
                raise PeerLost(r, f"{self.step - int(step_s)} steps behind")
