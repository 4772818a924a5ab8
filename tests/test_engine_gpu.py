"""Engine on a B200 in bf16 through the CUDA kernels, against the fp32 CPU oracle of the same model."""
import pytest
import torch

import flextrain_b200 as ft
from flextrain_b200.bench.naive import clone_params, naive_loss
from conftest import build_tiny

pytestmark = pytest.mark.gpu


def _copy_weights(src_am, dst_am):
    src = {(s, l, n): t for s, l, n, t in src_am.named_master_params()}
    for s, l, n, t in dst_am.named_master_params():
        t.copy_(src[(s, l, n)].to(t.dtype))


@pytest.mark.parametrize("attn_backend", ["auto", "library"])
def test_tiny_llama_bf16_tracks_fp32(attn_backend):
    from flextrain_b200 import ops
    ops.set_attention_backend(attn_backend)
    try:
        dims = dict(vocab_size=1024, n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, expert_dim=704,
                    ffn_dim=704, num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)
        cpu = build_tiny(dims=dims)
        gpu = build_tiny(dims=dims, device="cuda:0", dtype=torch.bfloat16,
                         optimizer=ft.AdamW(lr=1e-3, state_dtype=torch.float32))
        _copy_weights(cpu, gpu)
        src = ft.SyntheticTokenSource(1024, 128, seed=3)
        for step in range(3):
            seqs = src.get_sequences(256)
            a = cpu.fwd_bwd(seqs); cpu.step()
            b = gpu.fwd_bwd(seqs); gpu.step()
            assert abs(a.loss - b.loss) < 0.03, (step, a.loss, b.loss)
        from flextrain_b200.ops import cuda as k
        assert "gemm_tcgen05" in k._libs and "elementwise" in k._libs, "CUDA kernels were not used"
        assert all(v == 0 for v in k.device_error_words().values())
    finally:
        ops.set_attention_backend("auto")


def test_gradients_bf16_vs_autograd():
    dims = dict(vocab_size=512, n_layers=1, d_model=256, n_heads=2, n_kv_heads=1, head_dim=128, expert_dim=512,
                ffn_dim=512, num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)
    cpu = build_tiny(dims=dims)
    gpu = build_tiny(dims=dims, device="cuda:0", dtype=torch.bfloat16)
    _copy_weights(cpu, gpu)
    # use the bf16-rounded weights on both sides
    for (s, l, n, t), (_, _, _, g) in zip(cpu.named_master_params(), gpu.named_master_params()):
        t.copy_(g.float().cpu())
    seqs = ft.SyntheticTokenSource(512, 128, seed=5).get_sequences(256)
    P = clone_params(cpu)
    naive_loss(cpu, P, seqs).backward()
    gpu.fwd_bwd(seqs)
    bm = gpu.buffers
    for (scope, l, name), p in P.items():
        g = {"embed": bm.embed_grads(), "head": bm.head_grads()}.get(scope) or bm.grads(l)
        got = g["g_" + name[2:]].float().cpu()
        cos = torch.nn.functional.cosine_similarity(got.flatten(), p.grad.flatten(), dim=0)
        assert cos > 0.99, (scope, l, name, float(cos))


def test_smoke_entry():
    import __graft_entry__ as ge
    ge.smoke()


@pytest.mark.parametrize("seq_len,chunk", [(128, 256), (512, 128)])
def test_hybrid_gated_deltanet_bf16_tracks_fp32(seq_len, chunk):
    """Qwen3.5-style hybrid (linear-attention + full-attention layers) through the hand-written Gated DeltaNet CUDA
    kernels, single-chunk and with the recurrent / conv state carried across the chunks of one sequence."""
    dims = dict(vocab_size=1024, n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, expert_dim=512,
                ffn_dim=512, num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)
    hyper = {"layer_pattern": "1L1F", "gdn": {"n_k_heads": 2, "n_v_heads": 4, "head_k_dim": 64, "head_v_dim": 64}}
    kw = dict(arch="qwen3_5", dims=dims, hyper=hyper, max_seq_len=seq_len, batch_tokens=512,
              ws=ft.WorkingSetConfig.simple(max_seq_len=seq_len, max_global_batch_tokens=512, chunk=chunk,
                                            round_tokens=512))
    cpu = build_tiny(**kw)
    gpu = build_tiny(device="cuda:0", dtype=torch.bfloat16, optimizer=ft.AdamW(lr=1e-3, state_dtype=torch.float32),
                     **kw)
    _copy_weights(cpu, gpu)
    src = ft.SyntheticTokenSource(1024, seq_len, seed=9)
    for step in range(3):
        seqs = src.get_sequences(512)
        a = cpu.fwd_bwd(seqs); cpu.step()
        b = gpu.fwd_bwd(seqs); gpu.step()
        assert abs(a.loss - b.loss) < 0.04, (step, a.loss, b.loss)
    from flextrain_b200.ops import cuda as k
    assert "gdn" in k._libs and "seqmix" in k._libs, "Gated DeltaNet CUDA kernels were not used"


@pytest.mark.parametrize("arch", ["gemma2", "gemma3", "gemma4"])
def test_gemma_family_bf16_tracks_fp32(arch):
    """Gemma 2: attention and final-logit soft-caps.  Gemma 3: sandwich norms, per-head QK-norm, sliding + global layers with their own RoPE bases, GeGLU, tied scaled
    embedding; Gemma 4 adds the scale-free V norm, unit attention scale, proportional RoPE and the layer scalar."""
    dims = dict(vocab_size=1024, n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, expert_dim=704,
                ffn_dim=704, num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)
    kw = dict(arch=arch, dims=dims, hyper={"sliding_window": 32, "layer_pattern": "SF"})
    cpu = build_tiny(**kw)
    gpu = build_tiny(device="cuda:0", dtype=torch.bfloat16, optimizer=ft.AdamW(lr=1e-3, state_dtype=torch.float32),
                     **kw)
    torch.manual_seed(4)
    for _, _, name, t in cpu.named_master_params():
        if "norm" in name or "scalar" in name:
            t.add_(torch.randn_like(t) * 0.1)
    _copy_weights(cpu, gpu)
    src = ft.SyntheticTokenSource(1024, 128, seed=17)
    for step in range(3):
        seqs = src.get_sequences(256)
        a = cpu.fwd_bwd(seqs); cpu.step()
        b = gpu.fwd_bwd(seqs); gpu.step()
        assert abs(a.loss - b.loss) < 0.04, (step, a.loss, b.loss)


@pytest.mark.parametrize("ws_kw,force", [
    (dict(chunk=128, host_act_buffer_size=256 << 20, n_gpu_act_slots=3), None),     # DP-solver tiers, host arena
    (dict(chunk=128, host_act_buffer_size=256 << 20), 0),                           # everything offloaded at tier 0
    (dict(chunk=128, n_gpu_layers=2, n_gpu_grads=2, n_gpu_opt_layers=2), None),     # weight / grad / opt rings
])
def test_long_sequence_with_host_offload_bf16_tracks_fp32(ws_kw, force):
    """One sequence spanning four chunks (rolling KV window) with activations and states streamed through pinned host
    memory on the side streams: the bf16 GPU run must follow the fp32 CPU run (a stream-ordering bug shows as NaN or
    drift here, not on the CPU where everything is synchronous)."""
    dims = dict(vocab_size=1024, n_layers=4, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, expert_dim=704,
                ffn_dim=704, num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)
    mk = lambda **kw: build_tiny(dims=dims, max_seq_len=512, batch_tokens=1024, force_saved_act_level=force,
                                 ws=ft.WorkingSetConfig.simple(max_seq_len=512, max_global_batch_tokens=1024,
                                                               round_tokens=1024, **ws_kw), **kw)
    cpu = mk()
    gpu = mk(device="cuda:0", dtype=torch.bfloat16, optimizer=ft.AdamW(lr=1e-3, state_dtype=torch.float32))
    _copy_weights(cpu, gpu)
    src = ft.SyntheticTokenSource(1024, 512, seed=13)
    for step in range(4):
        seqs = src.get_sequences(1024)
        a = cpu.fwd_bwd(seqs); cpu.step()
        b = gpu.fwd_bwd(seqs); gpu.step()
        assert abs(a.loss - b.loss) < 0.04, (step, a.loss, b.loss)
    gpu.destroy()


def test_multimodal_bf16_tracks_fp32(tmp_path):
    """Image + text sequences on the GPU (vision tower in bf16 through SDPA, MRoPE through the RoPE kernel, splice by
    index copy) against the fp32 CPU engine on the same tiny random vision-language checkpoint."""
    pytest.importorskip("transformers")
    from flextrain_b200.engine.host_memory import UnpinnedHostBackend
    from test_multimodal_cpu import _hf_vl_model, _mm_sequence, _save_hub_layout
    _save_hub_layout(_hf_vl_model(), str(tmp_path))
    common = dict(max_seq_len=128, max_global_batch_tokens=256, max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30,
                  enable_multimodal=True,
                  working_set=ft.WorkingSetConfig.simple(max_seq_len=128, max_global_batch_tokens=256, chunk=64,
                                                         round_tokens=256))
    cpu = ft.from_pretrained(str(tmp_path), optimizer=ft.AdamW(lr=1e-3, state_dtype=torch.float32), device="cpu",
                             compute_dtype=torch.float32, master_dtype=torch.float32, grad_dtype=torch.float32,
                             host_backend=UnpinnedHostBackend(), **common)
    gpu = ft.from_pretrained(str(tmp_path), optimizer=ft.AdamW(lr=1e-3, state_dtype=torch.float32), device="cuda:0",
                             **common)
    seqs = [_mm_sequence(0, [(1, 4, 6), (1, 8, 4)], 3, [5, 7, 60]), _mm_sequence(1, [(1, 4, 4)], 4, [11, 70]),
            _mm_sequence(2, [], 5, [40])]
    for step in range(3):
        a = cpu.fwd_bwd(seqs); cpu.step()
        b = gpu.fwd_bwd(seqs); gpu.step()
        assert abs(a.loss - b.loss) < 0.05, (step, a.loss, b.loss)
    assert gpu.embed.last_summary.n_images == 3


def test_lora_bf16_tracks_fp32_on_the_tensor_core_kernel(monkeypatch):
    """LoRA r=16 on every linear of a tiny Llama: the merged weight, both rank-r gradient products and the adapter
    update run on the hand-written GEMM (strict mode would raise on a library call); losses track the fp32 CPU run and
    only the adapters move."""
    from flextrain_b200 import ops
    monkeypatch.setenv("FTB_STRICT", "1")
    dims = dict(vocab_size=1024, n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=64, expert_dim=704,
                ffn_dim=704, num_routed_experts=0, num_shared_experts=0, top_k=0, is_causal=True)
    kw = dict(lora_targets="all", lora_rank=16, lora_alpha=32.0, lora_adapter_opt_state_dtype=torch.float32)
    cpu = build_tiny(dims=dims, lora_adapter_compute_dtype=torch.float32, lora_adapter_master_dtype=torch.float32,
                     lora_adapter_grad_dtype=torch.float32, **kw)
    gpu = build_tiny(dims=dims, device="cuda:0", dtype=torch.bfloat16,
                     optimizer=ft.AdamW(lr=1e-3, state_dtype=torch.float32), **kw)
    _copy_weights(cpu, gpu)
    base0 = {(s, l, n): t.clone() for s, l, n, t in gpu.named_master_params() if "_lora_" not in n}
    src = ft.SyntheticTokenSource(1024, 128, seed=3)
    ops.reset_backends_used()
    for step in range(4):
        seqs = src.get_sequences(256)
        a = cpu.fwd_bwd(seqs); cpu.step()
        b = gpu.fwd_bwd(seqs); gpu.step()
        assert abs(a.loss - b.loss) < 0.03, (step, a.loss, b.loss)
    assert ops.backends_used().get("gemm") == ["tcgen05"], ops.backends_used()
    moved = 0.0
    for s, l, n, t in gpu.named_master_params():
        if "_lora_b" in n:
            moved = max(moved, float(t.float().abs().max()))
        elif "_lora_" not in n:
            assert torch.equal(t, base0[(s, l, n)]), (s, l, n)
    assert moved > 0
    from flextrain_b200.ops import cuda as k
    assert all(v == 0 for v in k.device_error_words().values())
