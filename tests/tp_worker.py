"""Worker for test_tp_gpu.py (run under torch.distributed.run): fused AG->GEMM and GEMM->RS against NCCL + matmul."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flextrain_b200.parallel.tp import TensorParallel  # noqa: E402


def rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


def main():
    out_path = sys.argv[1]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = f"cuda:{local}"
    dist.init_process_group("nccl", device_id=torch.device(dev))
    tp = TensorParallel(rank, world, dev, None, backend="p2p")
    base = TensorParallel(rank, world, dev, None, backend="collective")
    torch.manual_seed(100 + rank)
    res = {}
    Tl, K, N = 256, 512, 384
    for it in range(3):                       # several calls: exercises the double-buffered staging
        x = (torch.randn(Tl, K, device=dev) * 0.5).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
        y = tp.ag_gemm(x, w)
        yw = base.ag_gemm(x, w)
        res[f"ag_{it}"] = rel(y, yw)
        wt = (torch.randn(K, N, device=dev) * 0.05).to(torch.bfloat16)       # MN-major B (dgrad layout)
        res[f"ag_nt_{it}"] = rel(tp.ag_gemm(x, wt, trans_w=False), base.ag_gemm(x, wt, trans_w=False))
        xa = (torch.randn(world * Tl, N, device=dev) * 0.5).to(torch.bfloat16)
        w2 = (torch.randn(K, N, device=dev) * 0.05).to(torch.bfloat16)
        r = (torch.randn(Tl, K, device=dev)).to(torch.bfloat16)
        z = tp.gemm_rs(xa, w2, residual_local=r)
        zw = base.gemm_rs(xa, w2, residual_local=r)
        res[f"rs_{it}"] = rel(z, zw)
    torch.cuda.synchronize()
    tp.group.check()
    from flextrain_b200.ops import cuda as k
    res["errors"] = k.device_error_words()
    if rank == 0:
        with open(out_path, "w") as f:
            json.dump(res, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
