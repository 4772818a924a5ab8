"""Symmetric peer-mapped memory for one NVSwitch box: one process per GPU.

``torch.distributed`` is used only as the bootstrap channel (exchange of 64-byte CUDA IPC handles)
and for the baseline path.  Every rank allocates the same-sized buffer with ``cudaMalloc``, opens
the peers' handles, and from then on kernels address ``ptrs[r] + offset`` directly — plain loads and
stores over NVLink, signalled with release/acquire flags that live in another symmetric buffer.
The reference project has no communication layer (single GPU); its only analogue is the
``HostMemoryBackend`` protocol, which anticipates remote memory (flextrain/engine/host_memory.py:1-36).
"""
from __future__ import annotations

import ctypes
from ctypes import c_double, c_int, c_void_p
from typing import List

import torch

MAX_RANKS = 8


class _RawCudaBuffer:
    """Exposes a raw device pointer through ``__cuda_array_interface__`` so torch can view it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class SymmetricBuffer:
    """A buffer that exists at the same size on every rank; ``ptrs[r]`` is rank r's copy mapped here."""

    def __init__(self, local: torch.Tensor, ptrs: List[int], owner=None, mc_ptr: int = 0):
        self.local = local
        self.ptrs = ptrs
        self.nbytes = local.numel()
        self._owner = owner
        self.c_ptrs = (c_void_p * len(ptrs))(*ptrs)
        self.mc_ptr = mc_ptr          # NVSwitch multicast address of the buffer (0: none; see PeerGroup.alloc)


class PeerGroup:
    def __init__(self, rank: int, world: int, device, process_group=None, num_flag_slots: int = 4096,
                 timeout_s: float = 30.0):
        import torch.distributed as dist
        from ..ops.cuda import load
        if world > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} ranks per box")
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.pg = process_group
        self.dist = dist
        self.lib = load("comm")
        self.timeout_s = timeout_s
        self._bufs: List[SymmetricBuffer] = []
        self._symm: List[SymmetricBuffer] = []
        self._raw: List[int] = []
        self.num_flag_slots = num_flag_slots
        self.flags = self.alloc(num_flag_slots * MAX_RANKS * 4)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.epoch = 0

    # ---------------------------------------------------------------- allocation
    def alloc(self, nbytes: int, multicast: bool = False) -> SymmetricBuffer:
        """``multicast=True`` allocates through ``torch.distributed._symmetric_memory`` (``cuMemCreate`` memory bound
        to an NVSwitch multicast object) so that kernels can reduce or broadcast in the switch with ``multimem.*``
        on ``buf.mc_ptr``; the peers' copies are mapped as well, so everything that works on ``ptrs`` still does.
        Falls back to the plain peer mapping when the platform reports no multicast support."""
        nbytes = (max(int(nbytes), 16) + 255) // 256 * 256
        sizes = [None] * self.world
        self.dist.all_gather_object(sizes, nbytes, group=self.pg)
        if any(s != nbytes for s in sizes):
            raise RuntimeError(f"symmetric allocation sizes differ across ranks: {sizes}")
        if multicast:
            buf = self._alloc_multicast(nbytes)
            if buf is not None:
                return buf
        with torch.cuda.device(self.device):
            p = c_void_p()
            rc = self.lib.ftb_comm_alloc(ctypes.byref(p), ctypes.c_size_t(nbytes))
            if rc != 0:
                raise MemoryError(f"cudaMalloc of {nbytes} bytes failed ({rc})")
            handle = ctypes.create_string_buffer(64)
            rc = self.lib.ftb_comm_ipc_get(p, handle)
            if rc != 0:
                raise RuntimeError(f"cudaIpcGetMemHandle failed ({rc})")
            handles = [None] * self.world
            self.dist.all_gather_object(handles, bytes(handle.raw), group=self.pg)
            ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    ptrs.append(p.value)
                    continue
                q = c_void_p()
                rc = self.lib.ftb_comm_ipc_open(ctypes.create_string_buffer(h, 64), ctypes.byref(q))
                if rc != 0:
                    raise RuntimeError(f"cudaIpcOpenMemHandle for rank {r} failed ({rc})")
                ptrs.append(q.value)
            local = torch.as_tensor(_RawCudaBuffer(p.value, nbytes), device=self.device)
        buf = SymmetricBuffer(local, ptrs, self)
        self._bufs.append(buf)
        self._raw.append(p.value)
        self.dist.barrier(group=self.pg)
        return buf

    def _alloc_multicast(self, nbytes: int):
        """Symmetric buffer bound to an NVSwitch multicast object, or ``None`` when this platform / PyTorch build cannot
        provide one (every rank then takes the plain peer mapping: the ranks agree on the outcome first)."""
        buf, err = None, None
        try:
            import torch.distributed._symmetric_memory as symm
            with torch.cuda.device(self.device):
                t = symm.empty(nbytes, dtype=torch.uint8, device=self.device)
                hdl = symm.rendezvous(t, group=self.pg if self.pg is not None else self.dist.group.WORLD)
            mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
            if mc:
                t.zero_()
                buf = SymmetricBuffer(t, [int(p) for p in hdl.buffer_ptrs], (self, hdl), mc_ptr=mc)
        except Exception as e:                       # this PyTorch or this fabric has no symmetric-memory support
            err = e
        oks = [None] * self.world
        self.dist.all_gather_object(oks, buf is not None, group=self.pg)
        if not all(oks):
            return None
        self._symm.append(buf)                       # torch owns and frees these
        self.dist.barrier(group=self.pg)
        return buf

    # ------------------------------------------------------------------ signalling
    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def signal_wait(self, slot: int, epoch: int, stream=None) -> None:
        """Store ``epoch`` into every peer's flag ``[slot][rank]`` and wait (bounded) for all peers' flags."""
        s = stream or torch.cuda.current_stream(self.device)
        rc = self.lib.ftb_comm_signal_wait(self.flags.c_ptrs, c_int(slot % self.num_flag_slots), c_int(self.rank),
                                           c_int(self.world), c_int(epoch), c_double(self.timeout_s),
                                           c_void_p(self.status.data_ptr()), c_void_p(s.cuda_stream))
        if rc != 0:
            raise RuntimeError(f"ftb_comm_signal_wait failed ({rc})")

    def check(self) -> None:
        """Host-side check after a step: raises if any bounded wait ran out (a peer never signalled)."""
        st = int(self.status.item())
        if st != 0:
            self.status.zero_()
            raise RuntimeError(f"rank {self.rank}: wait for peer {st - 1} timed out after {self.timeout_s}s")

    def close(self) -> None:
        for b in self._bufs:
            for r, p in enumerate(b.ptrs):
                if r != self.rank:
                    self.lib.ftb_comm_ipc_close(c_void_p(p))
        for p in self._raw:
            self.lib.ftb_comm_free(c_void_p(p))
        self._bufs.clear(); self._raw.clear()


def shard_range(n: int, rank: int, world: int, quantum: int = 8):
    """Element range of ``rank`` in a segment of ``n`` elements, split in multiples of ``quantum``."""
    per = (n + quantum * world - 1) // (quantum * world) * quantum
    begin = min(n, rank * per)
    return begin, min(n, begin + per) - begin
