"""Small, self-terminating kernel cases for profiling one kernel at a time.

    python -m flextrain_b200.bench.kernel_cases gemm_fwd|gemm_dgrad|gemm_wgrad|rmsnorm_bwd|softmax_ce|attn_fwd|attn_bwd|
                                                  attn_fwd_one_tile|attn_bwd_unordered|attn_bwd_thread_reds|attn_fwd_32k|attn_bwd_32k|attn_bwd_32k_thread_reds|gdn_fwd|gdn_bwd|
                                                  gdn_long_fwd|rope|ffn_glu_fwd|ffn_glu_bwd|moe_grouped_gemm|moe_grouped_wgrad|moe_plan|gdn_fla_fwd|attn_fa2_fwd|attn_fa2_bwd|attn_fa2_fwd_32k|attn_fa2_bwd_32k

Each case holds a few hundred MB on the device (inputs larger than the 126 MB L2), runs three warm-up launches and
ten timed launches with CUDA events, and prints achieved TFLOP/s or GB/s.  They are the commands behind the
summaries in ``profiles/``.
"""
from __future__ import annotations

import sys

import torch


def _time(fn, n=10, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n


def main(case: str) -> None:
    from flextrain_b200 import ops
    from flextrain_b200.ops import cuda as k
    dev = "cuda"
    bf = torch.bfloat16
    if case.startswith("gemm"):
        M, N, K = 8192, 8192, 4096
        ta, tb = {"gemm_fwd": (False, True), "gemm_dgrad": (False, False), "gemm_wgrad": (True, False)}[case]
        a = torch.randn((K, M) if ta else (M, K), device=dev, dtype=bf)
        b = torch.randn((N, K) if tb else (K, N), device=dev, dtype=bf)
        out = torch.empty(M, N, device=dev, dtype=bf)
        ms = _time(lambda: k.gemm(a, b, trans_a=ta, trans_b=tb, out=out))
        print(f"{case}: M={M} N={N} K={K}  {ms:.3f} ms  {2.0 * M * N * K / ms / 1e9:.0f} TFLOP/s")
    elif case == "rmsnorm_bwd":
        T, D = 16384, 4096
        x, dy, res = (torch.randn(T, D, device=dev, dtype=bf) for _ in range(3))
        w = torch.ones(D, device=dev)
        _, r = k.rmsnorm_fwd(x, w, 1e-5)
        dw = torch.zeros(D, device=dev)
        ms = _time(lambda: k.rmsnorm_bwd(dy, x, w, r, dx_add=res, emit_y=True, dw_out=dw))
        print(f"{case}: T={T} D={D}  {ms:.3f} ms  {5.0 * T * D * 2 / ms / 1e6:.0f} GB/s (3 reads + 2 writes)")
    elif case == "softmax_ce":
        T, V = 2048, 128256
        z = torch.randn(T, V, device=dev, dtype=bf)
        tgt = torch.randint(0, V, (T,), device=dev)
        ms = _time(lambda: k.softmax_ce_(z, tgt, grad_scale=1e-3))
        print(f"{case}: T={T} V={V}  {ms:.3f} ms  {3.0 * T * V * 2 / ms / 1e6:.0f} GB/s (2 reads + 1 write)")
    elif case == "gdn_fla_fwd":
        # Third-party bar for the Gated DeltaNet kernels: flash-linear-attention's chunked Triton kernels (the ones the
        # reference calls, flextrain/nn/blocks/linear_attn.py:1036-1046) on the same shape as gdn_fwd.  A measurement
        # only: nothing in the package imports fla.  (Forward only: FLA's backward raised a misaligned-address fault
        # inside its own kernels on this hardware, so it is not run.)
        import torch.nn.functional as F
        from fla.ops.gated_delta_rule import chunk_gated_delta_rule
        HK, HV, dk, dv, S, L = 16, 32, 128, 128, 16, 1024
        T = S * L
        rep = HV // HK
        q = F.normalize(torch.randn(1, T, HK, dk, device=dev), dim=-1).to(bf).repeat_interleave(rep, 2)
        kk = F.normalize(torch.randn(1, T, HK, dk, device=dev), dim=-1).to(bf).repeat_interleave(rep, 2)
        v = (torch.randn(1, T, HV, dv, device=dev) * 0.5).to(bf)
        g = (-torch.rand(1, T, HV, device=dev) * 0.3).contiguous()
        beta = (torch.rand(1, T, HV, device=dev) * 0.9 + 0.05).to(bf).contiguous()
        cu = torch.arange(0, T + 1, L, device=dev, dtype=torch.long)
        fl = 2.0 * T * HV * dk * dv * 3
        with torch.no_grad():
            ms = _time(lambda: chunk_gated_delta_rule(q, kk, v, g, beta, cu_seqlens=cu, output_final_state=True))
        print(f"{case}: {S} x {L} tokens, HV={HV} dk={dk} dv={dv}  {ms:.3f} ms (FLA chunked Triton forward)")
        print("device error words: {}")
        return
    elif case in ("gdn_fwd", "gdn_bwd", "gdn_long_fwd"):
        import torch.nn.functional as F
        from flextrain_b200.ops import linattn_cuda as la
        # Qwen3.5-9B linear-attention shape: 16 key heads, 32 value heads, 128 x 128 state per head
        HK, HV, dk, dv = 16, 32, 128, 128
        S, L = (1, 16384) if case == "gdn_long_fwd" else (16, 1024)
        T = S * L
        q = F.normalize(torch.randn(T, HK, dk, device=dev), dim=-1).to(bf)
        kk = F.normalize(torch.randn(T, HK, dk, device=dev), dim=-1).to(bf)
        v = (torch.randn(T, HV, dv, device=dev) * 0.5).to(bf)
        g = (-torch.rand(T, HV, device=dev) * 0.3).contiguous()
        beta = (torch.rand(T, HV, device=dev) * 0.9 + 0.05).contiguous()
        cu = torch.arange(0, T + 1, L, device=dev, dtype=torch.int32)
        fl = 2.0 * T * HV * dk * dv * 3          # decay+predict, update, read-out: 3 multiply-adds per state element
        if case != "gdn_bwd":
            ms = _time(lambda: la.gdn_fwd(q, kk, v, g, beta, cu, None, want_r=True))
            print(f"{case}: {S} x {L} tokens, HV={HV} dk={dk} dv={dv}  {ms:.3f} ms  {fl / ms / 1e9:.1f} TFLOP/s fp32 "
                  f"(state recurrence on CUDA cores)")
        else:
            o, fin, r = la.gdn_fwd(q, kk, v, g, beta, cu, None, want_r=True)
            d_o = torch.randn_like(o)
            ms = _time(lambda: la.gdn_bwd(q, kk, v, g, beta, cu, None, fin, r, d_o))
            print(f"{case}: {S} x {L} tokens, HV={HV} dk={dk} dv={dv}  {ms:.3f} ms  {2.2 * fl / ms / 1e9:.1f} TFLOP/s fp32")
    elif case in ("attn_fwd", "attn_bwd", "attn_bwd_unordered", "attn_fwd_one_tile", "attn_fwd_32k", "attn_bwd_32k",
                  "attn_bwd_thread_reds", "attn_bwd_32k_thread_reds"):
        if case.endswith("_thread_reds"):      # dQ by per-thread 16-byte reductions (the earlier drain), same GPU
            k.load("attention").ftb_attn_set_dq_bulk(0)
            case = case[: -len("_thread_reds")]
        S, B, H, KV, hd = (32768, 1, 32, 8, 128) if case.endswith("_32k") else (1024, 16, 32, 8, 128)
        if case == "attn_fwd_one_tile":          # the one-query-tile-per-CTA forward kernel, for an A/B on the same GPU
            k.load("attention").ftb_attn_set_two_tiles(0)
            case = "attn_fwd"
        T = S * B
        q = torch.randn(T, H, hd, device=dev, dtype=bf)
        kk = torch.randn(T, KV, hd, device=dev, dtype=bf)
        v = torch.randn(T, KV, hd, device=dev, dtype=bf)
        cu = torch.arange(0, T + 1, S, device=dev, dtype=torch.int32)
        fl = 4.0 * B * H * S * S * hd / 2
        if case.startswith("attn_fwd"):
            ms = _time(lambda: ops.attention_fwd(q, kk, v, cu, cu, S, S, scale=hd ** -0.5))
            print(f"{case}: B={B} S={S} H={H} KV={KV} hd={hd}  {ms:.3f} ms  {fl / ms / 1e9:.0f} TFLOP/s (causal)")
        else:
            import os
            if case == "attn_bwd_unordered":       # dQ added in whatever order the CTAs arrive (not reproducible)
                os.environ["FTB_ATTN_DETERMINISTIC"] = "0"
            o, lse = ops.attention_fwd(q, kk, v, cu, cu, S, S, scale=hd ** -0.5)
            do = torch.randn_like(o)
            ms = _time(lambda: ops.attention_bwd(do, q, kk, v, o, lse, cu, cu, S, S, scale=hd ** -0.5))
            print(f"{case}: B={B} S={S} H={H} KV={KV} hd={hd}  {ms:.3f} ms  {2.5 * fl / ms / 1e9:.0f} TFLOP/s (causal)")
    elif case in ("attn_fa2_fwd", "attn_fa2_bwd", "attn_fa2_fwd_32k", "attn_fa2_bwd_32k"):
        # Third-party bar: flash_attn 2.8 (the package in this image; mma.sync kernels recompiled for sm_100) on the same
        # problems as attn_fwd / attn_bwd, deterministic backward as the reference asks of it.  A measurement only.
        from flash_attn import flash_attn_varlen_func
        S, B, H, KV, hd = (32768, 1, 32, 8, 128) if case.endswith("_32k") else (1024, 16, 32, 8, 128)
        T = S * B
        q = torch.randn(T, H, hd, device=dev, dtype=bf, requires_grad=True)
        kk = torch.randn(T, KV, hd, device=dev, dtype=bf, requires_grad=True)
        v = torch.randn(T, KV, hd, device=dev, dtype=bf, requires_grad=True)
        cu = torch.arange(0, T + 1, S, device=dev, dtype=torch.int32)
        fl = 4.0 * B * H * S * S * hd / 2
        run = lambda: flash_attn_varlen_func(q, kk, v, cu, cu, S, S, causal=True, deterministic=True)
        if "_fwd" in case:
            with torch.no_grad():
                ms = _time(run)
            print(f"{case}: B={B} S={S} H={H} KV={KV} hd={hd}  {ms:.3f} ms  {fl / ms / 1e9:.0f} TFLOP/s (causal, flash_attn 2)")
        else:
            o = run()
            do = torch.randn_like(o)
            ms = _time(lambda: torch.autograd.grad(o, (q, kk, v), do, retain_graph=True))
            print(f"{case}: B={B} S={S} H={H} KV={KV} hd={hd}  {ms:.3f} ms  {2.5 * fl / ms / 1e9:.0f} TFLOP/s "
                  f"(causal, flash_attn 2 backward only)")
        print("device error words: {}")
        return
    elif case == "rope":
        T, H, hd = 16384, 32, 128
        x = torch.randn(T, H, hd, device=dev, dtype=bf)
        pos = torch.arange(T, device=dev, dtype=torch.int32) % 1024
        inv = ops.rope_inv_freq(hd, 5e5).to(dev)
        ms = _time(lambda: ops.rope(x, pos, inv))
        print(f"{case}: T={T} H={H} hd={hd}  {ms:.3f} ms  {2.0 * T * H * hd * 2 / ms / 1e6:.0f} GB/s (1 read + 1 write)")
    elif case in ("moe_grouped_gemm", "moe_grouped_wgrad", "moe_plan"):
        # Qwen3-30B-A3B expert shapes: 128 experts, d 2048, expert width 768, top-8 routing of one 16,384-token chunk
        E, D, F, T, K = 128, 2048, 768, 16384, 8
        torch.manual_seed(3)
        logits = torch.randn(T, E, device=dev)
        experts = logits.topk(K, dim=1).indices.to(torch.int32)
        if case == "moe_plan":
            ms = _time(lambda: ops.moe_plan(experts, E, 64))
            print(f"{case}: T={T} K={K} E={E}  {ms:.3f} ms (histogram + scan + map kernels, no host read)")
        else:
            plan = ops.moe_plan(experts, E, 64)
            R = int(plan.rows)
            x = torch.randn(R, D, device=dev, dtype=bf) * 0.5
            w = torch.randn(E, 2 * F, D, device=dev, dtype=bf) * D ** -0.5
            if case == "moe_grouped_gemm":
                out = torch.empty(R, 2 * F, device=dev, dtype=bf)
                ms = _time(lambda: k.grouped_gemm(x, w, plan.offsets, out=out))
                print(f"{case}: rows={R} E={E} N={2 * F} K={D}  {ms:.3f} ms  {2.0 * T * K * 2 * F * D / ms / 1e9:.0f} "
                      f"TFLOP/s (useful rows)")
            else:
                dy = torch.randn(R, 2 * F, device=dev, dtype=bf) * 0.1
                gw = torch.zeros(E, 2 * F, D, device=dev, dtype=bf)
                ms = _time(lambda: k.grouped_wgrad(dy, x, plan.offsets, gw))
                print(f"{case}: rows={R} E={E} N={2 * F} K={D}  {ms:.3f} ms  {2.0 * T * K * 2 * F * D / ms / 1e9:.0f} "
                      f"TFLOP/s (useful rows)")
    elif case in ("ffn_glu_fwd", "ffn_glu_bwd"):
        # Llama-3.1-8B gated FFN on one 16,384-token chunk: fused GEMM + activation epilogue against GEMM then activation
        M, K, F = 16384, 4096, 14336
        x = torch.randn(M, K, device=dev, dtype=bf) * 0.5
        w13 = torch.randn(2 * F, K, device=dev, dtype=bf) * K ** -0.5
        w2 = torch.randn(K, F, device=dev, dtype=bf) * F ** -0.5
        x13 = torch.empty(M, 2 * F, device=dev, dtype=bf)
        if case == "ffn_glu_fwd":
            fused = _time(lambda: k.gemm_glu_fwd(x, w13, "swiglu", x13=x13))
            def two():
                k.gemm(x, w13, trans_b=True, out=x13)
                k.glu_fwd(x13[:, :F], x13[:, F:], "swiglu")
            fl = 2.0 * M * K * 2 * F
        else:
            k.gemm(x, w13, trans_b=True, out=x13)
            dx13 = torch.empty_like(x13)
            fused = _time(lambda: k.gemm_glu_bwd(x, w2, x13, "swiglu", dx13=dx13))
            def two():
                dact = k.gemm(x, w2)
                k.glu_bwd(dact, x13[:, :F], x13[:, F:], "swiglu", dgate=dx13[:, :F], dup=dx13[:, F:])
            fl = 2.0 * M * K * F
        sep = _time(two)
        print(f"{case}: M={M} K={K} F={F}  fused {fused:.3f} ms ({fl / fused / 1e9:.0f} TFLOP/s)  "
              f"GEMM + activation pass {sep:.3f} ms")
    else:
        raise SystemExit(f"unknown case {case}")
    print("device error words:", k.device_error_words())


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else "gemm_fwd")
