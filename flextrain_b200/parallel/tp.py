"""Tensor parallelism with sequence-parallel activations: fused all-gather→GEMM and GEMM→reduce-scatter.

Activations between blocks are token-sharded ``(T/tp, d)``.  A column-parallel projection needs the full token
range (all-gather) and a row-parallel projection produces partial sums for all tokens (reduce-scatter):

``ag_gemm``   ``y (T, N_local) = allgather(x_local) @ w_local.T`` in ONE kernel: the tcgen05 GEMM starts on the local
              row panel while two extra warps per CTA pull the peers' panels over NVLink into local HBM and publish
              per-panel arrival counters that gate the TMA producer (``csrc/gemm_tcgen05.cu``, comm mode 1).
``gemm_rs``   ``y_local (T/tp, N) = reduce_scatter(x @ w_local.T)``: the GEMM epilogue stores every partial output tile
              straight into its owner's staging slot (peer stores, tile by tile under the math, comm mode 2), then a
              flag exchange and a slot-sum kernel (+ residual) finish on the owner.

Staging buffers are double-buffered so a rank may fill its next panel while peers still read the previous one; each
call begins with a flag exchange.  ``backend="collective"`` is the library baseline (all_gather / reduce_scatter +
plain GEMM) and the CPU path.  The reference project has no tensor parallelism.
"""
from __future__ import annotations

from ctypes import c_float, c_int, c_long, c_void_p
from typing import Dict, Optional, Tuple

import torch

from .. import ops


class TensorParallel:
    def __init__(self, rank: int, world: int, device, process_group=None, backend: str = "p2p", group=None):
        self.rank, self.world, self.device, self.pg, self.backend = rank, world, torch.device(device), process_group, backend
        self.group = group
        if backend == "p2p" and group is None:
            from .comm import PeerGroup
            self.group = PeerGroup(rank, world, device, process_group)
        self._ag: Dict[Tuple[int, int], list] = {}
        self._rs: Dict[Tuple[int, int], list] = {}
        self._calls = 0
        self._counter = None
        self.slot_base = 3000

    # ----------------------------------------------------------------- staging
    def _ag_stage(self, rows: int, K: int):
        key = (rows, K)
        if key not in self._ag:
            self._ag[key] = [self.group.alloc(rows * K * 2) for _ in range(2)]
        return self._ag[key]

    def _rs_stage(self, panel_rows: int, N: int):
        key = (panel_rows, N)
        if key not in self._rs:
            self._rs[key] = [self.group.alloc(self.world * panel_rows * N * 2) for _ in range(2)]
        return self._rs[key]

    def _sync(self) -> None:
        self.group.signal_wait(self.slot_base + (self._calls % 64), self.group.next_epoch())
        self._calls += 1

    # ------------------------------------------------------------------- ops
    def ag_gemm(self, x_local: torch.Tensor, w_local: torch.Tensor, *, trans_w: bool = True) -> torch.Tensor:
        """``allgather_tokens(x_local) @ (w_local.T if trans_w else w_local)``; ``x_local (T/tp, K)`` bf16."""
        Tl, K = x_local.shape
        W = self.world
        if self.backend != "p2p":
            import torch.distributed as dist
            full = torch.empty(W * Tl, K, dtype=x_local.dtype, device=x_local.device)
            dist.all_gather_into_tensor(full, x_local.contiguous(), group=self.pg)
            self.last_gathered = full
            return ops.gemm(full, w_local, trans_b=trans_w)
        assert Tl % 128 == 0 and x_local.dtype == torch.bfloat16
        bufs = self._ag_stage(W * Tl, K)
        buf = bufs[self._calls % 2]
        stage = buf.local.view(torch.bfloat16)[: W * Tl * K].view(W * Tl, K)
        stage[self.rank * Tl:(self.rank + 1) * Tl].copy_(x_local)
        self._sync()                                     # every rank's panel is in place; previous readers are done
        if self._counter is None:
            self._counter = torch.zeros(8, dtype=torch.int64, device=self.device)
        self._counter.zero_()
        N = w_local.shape[0] if trans_w else w_local.shape[1]
        out = torch.empty(W * Tl, N, dtype=torch.bfloat16, device=self.device)
        lib = self.group.lib if hasattr(self.group.lib, "ftb_gemm_bf16_tp") else None
        from ..ops.cuda import load, _stream
        g = load("gemm_tcgen05")
        rc = g.ftb_gemm_bf16_tp(c_int(1), c_void_p(stage.data_ptr()), buf.c_ptrs, c_void_p(self._counter.data_ptr()),
                                c_void_p(w_local.data_ptr()), c_void_p(out.data_ptr()), None, c_long(0),
                                c_int(W * Tl), c_int(N), c_int(K), c_int(0 if trans_w else 1), c_int(K),
                                c_int(w_local.stride(0)), c_int(N), c_float(1.0), c_int(0), c_int(W), c_int(self.rank),
                                c_int(0), _stream())
        if rc != 0:
            raise RuntimeError(f"ftb_gemm_bf16_tp(ag) failed ({rc})")
        ops._count()
        self.last_gathered = stage
        return out

    def gemm_rs(self, x: torch.Tensor, w_local: torch.Tensor, *, trans_w: bool = True,
                residual_local: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``reduce_scatter_tokens(x @ w_local.T) (+ residual_local)``; ``x (T, K_local)`` bf16 → ``(T/tp, N)``."""
        T, K = x.shape
        W = self.world
        N = w_local.shape[0] if trans_w else w_local.shape[1]
        Tl = T // W
        if self.backend != "p2p":
            import torch.distributed as dist
            part = ops.gemm(x, w_local, trans_b=trans_w)
            out = torch.empty(Tl, N, dtype=part.dtype, device=part.device)
            if dist.get_backend(self.pg) == "gloo":
                dist.all_reduce(part, group=self.pg)
                out.copy_(part[self.rank * Tl:(self.rank + 1) * Tl])
            else:
                dist.reduce_scatter_tensor(out, part, group=self.pg)
            return out if residual_local is None else out + residual_local
        assert Tl % 128 == 0 and x.dtype == torch.bfloat16
        bufs = self._rs_stage(Tl, N)
        buf = bufs[self._calls % 2]
        from ..ops.cuda import load, _stream
        g = load("gemm_tcgen05")
        rc = g.ftb_gemm_bf16_tp(c_int(2), c_void_p(x.data_ptr()), None, None, c_void_p(w_local.data_ptr()), None,
                                buf.c_ptrs, c_long(Tl * N), c_int(T), c_int(N), c_int(K), c_int(0 if trans_w else 1),
                                c_int(x.stride(0)), c_int(w_local.stride(0)), c_int(N), c_float(1.0), c_int(0),
                                c_int(W), c_int(self.rank), c_int(0), _stream())
        if rc != 0:
            raise RuntimeError(f"ftb_gemm_bf16_tp(rs) failed ({rc})")
        ops._count()
        self._sync()                                     # all partial panels have landed in my slots
        out = torch.empty(Tl, N, dtype=torch.bfloat16, device=self.device)
        rc = self.group.lib.ftb_comm_reduce_slots(c_void_p(buf.local.data_ptr()), c_long(Tl * N), c_int(W),
                                                  c_void_p(residual_local.data_ptr() if residual_local is not None else 0),
                                                  c_void_p(out.data_ptr()), c_long(Tl * N), _stream())
        if rc != 0:
            raise RuntimeError(f"ftb_comm_reduce_slots failed ({rc})")
        ops._count()
        return out

    def all_gather(self, x_local: torch.Tensor) -> torch.Tensor:
        """Token all-gather ``(T/tp, ...) -> (T, ...)`` (rank-major) for the operands of weight gradients and for
        per-token results.  Peer path: each rank stores its part into every peer's staging buffer."""
        W = self.world
        x_local = x_local.contiguous()
        if self.backend != "p2p":
            import torch.distributed as dist
            full = torch.empty((W * x_local.shape[0],) + tuple(x_local.shape[1:]), dtype=x_local.dtype,
                               device=x_local.device)
            dist.all_gather_into_tensor(full, x_local, group=self.pg)
            return full
        nb = x_local.numel() * x_local.element_size()
        assert nb % 16 == 0, "token all-gather moves 16-byte units"
        bufs = self._ag_stage(W * nb // 2, 1)              # staging is sized in bf16 elements
        buf = bufs[self._calls % 2]
        stage = buf.local[: W * nb]
        stage[self.rank * nb:(self.rank + 1) * nb].copy_(x_local.view(-1).view(torch.uint8))
        self._sync()                                     # previous readers of this staging buffer are done
        from ..ops.cuda import _stream
        rc = self.group.lib.ftb_comm_allgather_push(buf.c_ptrs, c_long(self.rank * nb), c_long(nb), c_int(W),
                                                    c_int(self.rank), _stream())
        if rc != 0:
            raise RuntimeError(f"ftb_comm_allgather_push failed ({rc})")
        ops._count()
        self._sync()                                     # every rank's part has landed here
        return stage.view(x_local.dtype).view((W * x_local.shape[0],) + tuple(x_local.shape[1:]))

    def all_reduce_(self, t: torch.Tensor) -> torch.Tensor:
        """Small replicated-gradient reduction (norm weights under sequence parallelism); library call."""
        import torch.distributed as dist
        dist.all_reduce(t, group=self.pg)
        return t
