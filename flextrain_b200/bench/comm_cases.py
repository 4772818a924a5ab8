"""Micro-benchmarks of the fused compute+collective paths against their rooflines and the library (NCCL) baselines.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        -m flextrain_b200.bench.comm_cases [out.json]

Paths (all kernels of ``csrc/comm.cu``, ``csrc/gemm_tcgen05.cu``, ``csrc/moe.cu``; device-timed with CUDA events,
max over ranks, 3 warm-up + 10 timed calls each):

  dp_reduce_scatter   fused gradient reduce-scatter + bf16->fp32 cast/scale over peer memory   vs  NCCL reduce_scatter + cast
  dp_adamw_push       sharded AdamW whose stores are the parameter all-gather                  vs  local AdamW + NCCL all_gather
  dp_param_gather_gemm parameter all-gather of a layer fused into its QKV projection            vs  NCCL all_gather x2 + GEMM
  tp_ag_gemm          all-gather -> GEMM in one kernel                                          vs  NCCL all_gather + GEMM
  tp_gemm_rs          GEMM -> reduce-scatter (peer-store epilogue + slot sum)                   vs  GEMM + NCCL reduce_scatter
  ep_dispatch         MoE token dispatch (peer stores into the owners' expert-major buffers)    vs  NCCL all_to_all (equal splits)
  ep_combine          weighted K-way combine (peer loads)                                        vs  NCCL all_to_all + local combine

Roofline of a path = the slower of (FLOPs / measured cuBLAS bf16 burst throughput) and (bytes that must cross NVLink per
GPU / 770 GB/s, the measured peer-copy bandwidth per direction); the table prints achieved = roofline time / measured time.
"""
from __future__ import annotations

import json
import os
import sys
from ctypes import c_float, c_int, c_long, c_uint, c_void_p

import torch
import torch.distributed as dist

LINK_GBS = 770.0


def _peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["bf16_tflops"]), float(p["hbm_gbs"]), "measured"
    except Exception:
        return 1590.0, 6650.0, "fallback"


def main() -> None:
    from flextrain_b200 import ops
    from flextrain_b200.parallel.comm import PeerGroup, shard_range
    from flextrain_b200.parallel.ep import ExpertParallel
    from flextrain_b200.parallel.tp import TensorParallel
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    tflops, hbm, src = _peaks()
    res = {"world": world, "peaks": {"bf16_tflops": tflops, "hbm_gbs": hbm, "link_gbs": LINK_GBS, "source": src}}

    def timeit(fn, n=10, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def record(name, fused_ms, base_ms, flops, link_bytes, hbm_bytes=0.0):
        roof_ms = max(flops / (tflops * 1e12), link_bytes / (LINK_GBS * 1e9), hbm_bytes / (hbm * 1e9)) * 1e3
        res[name] = {"fused_ms": fused_ms, "library_ms": base_ms, "roofline_ms": roof_ms,
                     "fraction_of_roofline": roof_ms / fused_ms, "speedup_vs_library": base_ms / fused_ms,
                     "flops": flops, "nvlink_bytes_per_gpu": link_bytes}

    group = PeerGroup(rank, world, dev, None)
    lib = group.lib
    stream = lambda: c_void_p(torch.cuda.current_stream().cuda_stream)

    # ------------------------------------------------------------------ (a) gradient reduce-scatter + cast/scale
    n = 1 << 28                                           # 256 Mi bf16 gradients = 512 MiB per rank
    gbuf = group.alloc(n * 2)
    gbuf.local.view(torch.bfloat16)[:n].normal_()
    beg, cnt = shard_range(n, rank, world)
    shard = torch.zeros(cnt + 8, dtype=torch.float32, device=dev)
    arr = lambda v, ct=c_long: (ct * 1)(v)
    slot = [0]

    def fused_rs():
        group.signal_wait(100 + slot[0] % 8, group.next_epoch()); slot[0] += 1
        rc = lib.ftb_comm_reduce_scatter(gbuf.c_ptrs, c_int(1), arr(0), arr(beg), arr(cnt), arr(0), arr(0, c_int),
                                         c_void_p(shard.data_ptr()), c_int(world), c_int(rank), c_float(0.5), stream())
        assert rc == 0, rc

    g_local = gbuf.local.view(torch.bfloat16)[:n]
    out_bf = torch.empty(n // world, dtype=torch.bfloat16, device=dev)

    def nccl_rs():
        dist.reduce_scatter_tensor(out_bf, g_local[: (n // world) * world])
        shard[: n // world].copy_(out_bf).mul_(0.5)

    record("dp_reduce_scatter", timeit(fused_rs), timeit(nccl_rs), 0.0, (world - 1) * cnt * 2,
           hbm_bytes=world * cnt * 2 + cnt * 4)

    # ------------------------------------------------------------------ (a') sharded AdamW + parameter all-gather
    pbuf = group.alloc(n * 2)
    pbuf.local.view(torch.bfloat16)[:n].normal_()
    m, v = torch.zeros_like(shard), torch.zeros_like(shard)

    def fused_adamw():
        rc = lib.ftb_comm_adamw_push(pbuf.c_ptrs, c_int(1), arr(0), arr(beg), arr(cnt), arr(0), arr(0, c_int),
                                     c_void_p(shard.data_ptr()), c_void_p(m.data_ptr()), c_void_p(v.data_ptr()),
                                     c_int(world), c_int(rank), c_float(1e-5), c_float(0.9), c_float(0.95),
                                     c_float(1e-8), c_float(0.0), c_float(0.1), c_float(0.05), c_uint(1), stream())
        assert rc == 0, rc
        group.signal_wait(110 + slot[0] % 8, group.next_epoch()); slot[0] += 1

    p_local = pbuf.local.view(torch.bfloat16)[:n]
    p_shard = p_local[beg:beg + cnt].clone()
    p_full = torch.empty(world * cnt, dtype=torch.bfloat16, device=dev)

    def nccl_adamw():
        ops.adamw_multi([p_shard], [shard[:cnt]], [m[:cnt]], [v[:cnt]], lrs=[1e-5], wds=[0.0], beta1=0.9, beta2=0.95,
                        eps=1e-8, step=3)
        dist.all_gather_into_tensor(p_full, p_shard)

    record("dp_adamw_push", timeit(fused_adamw), timeit(nccl_adamw), 0.0, (world - 1) * cnt * 2,
           hbm_bytes=cnt * (4 * 5 + 2 * 2))

    # ------------------------------------------------------------------ (c) tensor-parallel fused GEMMs (70B shapes)
    tp = TensorParallel(rank, world, dev, None, backend="p2p", group=group)
    base = TensorParallel(rank, world, dev, None, backend="collective")
    Tl, K, N = 16384 // world, 8192, 28672 // world
    x = (torch.randn(Tl, K, device=dev) * 0.5).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    xa = (torch.randn(world * Tl, N, device=dev) * 0.5).to(torch.bfloat16)
    w2 = (torch.randn(K, N, device=dev) * 0.05).to(torch.bfloat16)
    fl = 2.0 * world * Tl * K * N
    link = (world - 1) * Tl * K * 2
    t_lib = timeit(lambda: base.ag_gemm(x, w))
    record("tp_ag_gemm", timeit(lambda: tp.ag_gemm(x, w)), t_lib, fl, link)
    # the same kernel with the remote panels pulled by two warps of 16-byte loads instead of bulk copies (A/B switch)
    from flextrain_b200.ops.cuda import load as _load_gemm
    _load_gemm("gemm_tcgen05").ftb_gemm_set_tp_pull_threads(c_int(1))
    record("tp_ag_gemm_thread_pull", timeit(lambda: tp.ag_gemm(x, w)), t_lib, fl, link)
    _load_gemm("gemm_tcgen05").ftb_gemm_set_tp_pull_threads(c_int(0))
    record("tp_gemm_rs", timeit(lambda: tp.gemm_rs(xa, w2)), timeit(lambda: base.gemm_rs(xa, w2)), fl, link)

    # ------------------------------------------------------------------ (b) parameter all-gather -> first GEMM
    # Llama-3.1-8B layer: the QKV projection (6144 x 4096) sits at the start of the 10240 x 4096 [q|k|v|o] segment; the
    # kernel also gathers the FFN segment (3 x 14336 x 4096) of the layer while it computes.
    from flextrain_b200.ops.cuda import load as _load
    gl = _load("gemm_tcgen05")
    Kd, Nq, n0, n1 = 4096, 6144, 10240 * 4096, 3 * 14336 * 4096
    arena = group.alloc((n0 + n1) * 2)
    arena.local.view(torch.bfloat16)[: n0 + n1].normal_(0, 0.02)
    xq = (torch.randn(16384, Kd, device=dev) * 0.5).to(torch.bfloat16)
    wq = arena.local.view(torch.bfloat16)[: Nq * Kd].view(Nq, Kd)
    outq = torch.empty(16384, Nq, dtype=torch.bfloat16, device=dev)
    cnt8 = torch.zeros(8, dtype=torch.int64, device=dev)
    per_ = lambda nel: (nel + 8 * world - 1) // (8 * world) * 8
    arr2 = lambda vals, ct=c_long: (ct * 2)(*vals)

    def fused_wgather():
        group.signal_wait(120 + slot[0] % 8, group.next_epoch()); slot[0] += 1      # everyone's ranges are final
        cnt8.zero_()
        rc = gl.ftb_gemm_bf16_wgather(c_void_p(xq.data_ptr()), c_void_p(wq.data_ptr()), c_void_p(outq.data_ptr()),
                                      c_int(16384), c_int(Nq), c_int(Kd), c_int(Kd), c_int(Nq), c_float(1.0),
                                      arena.c_ptrs, c_int(2), arr2([0, n0 * 2]), arr2([n0, n1]), arr2([2, 2], c_int),
                                      arr2([per_(n0), per_(n1)]), c_void_p(cnt8.data_ptr()), c_int(world), c_int(rank),
                                      c_int(0), stream())
        assert rc == 0, rc

    flat = arena.local.view(torch.bfloat16)[: n0 + n1]
    sh0, sh1 = flat[:n0][rank * per_(n0):(rank + 1) * per_(n0)].clone(), flat[n0:][rank * per_(n1):(rank + 1) * per_(n1)].clone()
    full0 = torch.empty(world * sh0.numel(), dtype=torch.bfloat16, device=dev)
    full1 = torch.empty(world * sh1.numel(), dtype=torch.bfloat16, device=dev)

    def nccl_wgather():
        dist.all_gather_into_tensor(full0, sh0)
        dist.all_gather_into_tensor(full1, sh1)
        ops.gemm(xq, full0[: Nq * Kd].view(Nq, Kd), trans_b=True, out=outq)

    record("dp_param_gather_gemm", timeit(fused_wgather), timeit(nccl_wgather), 2.0 * 16384 * Nq * Kd,
           (n0 + n1) * 2 * (world - 1) / world)

    # ------------------------------------------------------------------ (d) expert-parallel dispatch / combine
    T, Kt, D, E = 16384, 8, 2048, 128
    ep = ExpertParallel(rank, world, dev, None, backend="p2p", group=group)
    torch.manual_seed(7 + rank)
    idx = torch.stack([torch.randperm(E, device=dev)[:Kt] for _ in range(64)]).repeat(T // 64, 1).to(torch.int32)
    wts = torch.rand(T, Kt, device=dev)
    h = torch.randn(T, D, device=dev).to(torch.bfloat16)
    cap = ep.capacity(T, Kt, E)
    plan = ep.plan(idx, wts, E)
    rows = max(plan.rows, 128)
    remote = T * Kt * D * 2 * (world - 1) / world         # bytes leaving (dispatch) / entering (combine) this GPU
    y = torch.randn(rows, D, device=dev).to(torch.bfloat16)
    # library baseline: gather the T x K routed rows into destination order, then one equal-split all-to-all
    send_order = torch.argsort(idx.reshape(-1).long(), stable=True) // Kt
    send = h[send_order].contiguous()
    recv_a2a = torch.empty_like(send)

    def nccl_dispatch():
        dist.all_to_all_single(recv_a2a, h[send_order])              # gather into send order + all-to-all

    def nccl_combine():
        dist.all_to_all_single(recv_a2a, send)
        (recv_a2a.view(T, Kt, D).float() * wts.unsqueeze(-1)).sum(1).to(torch.bfloat16)

    record("ep_dispatch", timeit(lambda: ep.dispatch(h, plan, cap, "recv_a")), timeit(nccl_dispatch), 0.0, remote)
    record("ep_combine", timeit(lambda: ep.combine(y, plan, wts, h, cap, "ybuf")), timeit(nccl_combine), 0.0, remote)

    torch.cuda.synchronize()
    group.check()
    from flextrain_b200.ops import cuda as k
    res["errors"] = k.device_error_words()
    if rank == 0:
        print(f"{'path':20s} {'fused ms':>9s} {'library ms':>11s} {'roofline ms':>12s} {'of roofline':>12s} {'vs library':>11s}")
        for name, r in res.items():
            if isinstance(r, dict) and "fused_ms" in r:
                print(f"{name:20s} {r['fused_ms']:9.3f} {r['library_ms']:11.3f} {r['roofline_ms']:12.3f} "
                      f"{r['fraction_of_roofline']:12.2f} {r['speedup_vs_library']:11.2f}")
        print("device error words:", res["errors"])
        if len(sys.argv) > 1:
            with open(sys.argv[1], "w") as f:
                json.dump(res, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
