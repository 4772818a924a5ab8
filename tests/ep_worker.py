"""Worker for the expert-parallel tests: W ranks, experts sharded, each rank routes its own tokens.  Compares the
EP forward / backward of one MoE block with a single-process evaluation of the same block over all ranks' tokens."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from flextrain_b200.core.activation_schema import ActivationSchema, ActivationSlot  # noqa: E402
from flextrain_b200.core.layer import LayerContext  # noqa: E402
from flextrain_b200.nn.blocks.ffn_moe import MoEConfig, MoEFFN  # noqa: E402
from flextrain_b200.parallel.ep import ExpertParallel  # noqa: E402


def run(rank, world, dev, backend, dtype, pg=None):
    torch.manual_seed(0)
    E, K, d, F, T = 8, 2, 128, 64, 256
    cfg = MoEConfig(d_model=d, num_experts=E, top_k=K, expert_dim=F)
    full = MoEFFN(cfg, dtype=dtype)
    P = {s.name: (torch.randn(s.shape) * 0.05).to(dtype).to(dev) for s in full.tensor_specs()}
    hs = [(torch.randn(T, d) * 0.5).to(dtype).to(dev) for _ in range(world)]
    dxs = [(torch.randn(T, d) * 0.1).to(dtype).to(dev) for _ in range(world)]
    # ---- reference: every rank evaluates the full block on all tokens (single-GPU code path)
    G = {"g_" + n[2:]: torch.zeros_like(p, dtype=torch.float32 if dtype == torch.float32 else dtype) for n, p in P.items()}
    outs, dhs = [], []
    sch = ActivationSchema(full.activation_fields())
    for r in range(world):
        slot = ActivationSlot(sch, T)
        ctx = LayerContext()
        outs.append(full.fwd(hs[r], hs[r], P, slot, ctx))
        dhs.append(full.bwd(dxs[r], hs[r], P, G, slot, ctx))
    # ---- expert parallel: local expert shard
    El = E // world
    ep = ExpertParallel(rank, world, dev, pg, backend=backend, capacity_factor=4.0)
    Pl = dict(P)
    Pl["w_up"] = P["w_up"][rank * El:(rank + 1) * El].contiguous()
    Pl["w_down"] = P["w_down"][rank * El:(rank + 1) * El].contiguous()
    Gl = {k: torch.zeros_like(v) for k, v in G.items()}
    Gl["g_up"] = torch.zeros_like(Pl["w_up"], dtype=G["g_up"].dtype)
    Gl["g_down"] = torch.zeros_like(Pl["w_down"], dtype=G["g_down"].dtype)
    slot = ActivationSlot(sch, T)
    ctx = LayerContext(ep=ep)
    out = full.fwd(hs[rank], hs[rank], Pl, slot, ctx)
    dh = full.bwd(dxs[rank], hs[rank], Pl, Gl, slot, ctx)
    ep.check()
    rel = lambda a, b: float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))
    res = {"out": rel(out, outs[rank]), "dh": rel(dh, dhs[rank]),
           "g_up": rel(Gl["g_up"], G["g_up"][rank * El:(rank + 1) * El]),
           "g_down": rel(Gl["g_down"], G["g_down"][rank * El:(rank + 1) * El])}
    # router gradient: the EP ranks each hold their own tokens' share; the sum over ranks is the reference
    gr = Gl["g_router"].float().clone()
    dist.all_reduce(gr, group=pg)
    res["g_router"] = rel(gr, G["g_router"])
    return res


def main():
    backend, out_path = sys.argv[1], sys.argv[2]
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    if backend == "p2p":
        torch.cuda.set_device(local)
        dev = f"cuda:{local}"
        dist.init_process_group("nccl", device_id=torch.device(dev))
        dtype = torch.bfloat16
    else:
        dev = "cpu"
        dist.init_process_group("gloo")
        dtype = torch.float32
    res = run(rank, world, dev, backend, dtype)
    allres = [None] * world
    dist.all_gather_object(allres, res)
    if rank == 0:
        worst = {k: max(r[k] for r in allres) for k in res}
        if backend == "p2p":
            from flextrain_b200.ops import cuda as k
            worst["errors"] = k.device_error_words()
        import json
        with open(out_path, "w") as f:
            json.dump(worst, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
