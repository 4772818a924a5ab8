"""Multimodal path on CPU against ``transformers``: image pre-processing, the vision tower, MRoPE position ids, and
the whole model (image + text -> loss and gradients) for a tiny random Qwen3.5 vision-language checkpoint
(the reference's analogues: tests/test_qwen_vl_vit_forward.py, tests/test_mrope_position_ids.py,
tests/test_concat_splice.py, tests/test_qwen3_5_mm_*.py)."""
import json
import os

import pytest
import torch

import flextrain_b200 as ft
from flextrain_b200.core.modality import ImageInputCPU
from flextrain_b200.engine.host_memory import UnpinnedHostBackend
from flextrain_b200.engine.schedule import compute_mrope_position_ids
from flextrain_b200.io.image_processing import (ImageGeometry, MultimodalProcessorBundle, build_multimodal_sequence,
                                                preprocess_frames, smart_resize)
from flextrain_b200.nn.encoders.qwen_vl_vit import QwenVLViT, ViTConfig
from flextrain_b200.nn.splices.concat import build_splice_maps, splice_backward, splice_forward

transformers = pytest.importorskip("transformers")

IMG, VID, VSTART, VEND = 300, 301, 302, 303
TEXT = dict(vocab_size=320, hidden_size=64, intermediate_size=112, num_hidden_layers=4, num_attention_heads=4,
            num_key_value_heads=2, head_dim=16, max_position_embeddings=512, rms_norm_eps=1e-5,
            tie_word_embeddings=False, linear_conv_kernel_dim=4, linear_key_head_dim=16, linear_value_head_dim=16,
            linear_num_key_heads=2, linear_num_value_heads=4, layer_types=["linear_attention", "full_attention"] * 2,
            rope_parameters={"rope_type": "default", "rope_theta": 10000.0, "partial_rotary_factor": 0.5,
                             "mrope_section": [2, 1, 1], "mrope_interleaved": True})
VISION = dict(depth=2, hidden_size=32, num_heads=2, intermediate_size=64, patch_size=4, temporal_patch_size=2,
              in_channels=3, spatial_merge_size=2, out_hidden_size=64, num_position_embeddings=64,
              hidden_act="gelu_pytorch_tanh")


def _hf_vl_model(moe: bool = False):
    if moe:
        text = {k: v for k, v in TEXT.items() if k != "intermediate_size"}
        text.update(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=48, shared_expert_intermediate_size=48)
        cfg = transformers.Qwen3_5MoeConfig(text_config=text, vision_config=dict(VISION), image_token_id=IMG,
                                            video_token_id=VID, vision_start_token_id=VSTART,
                                            vision_end_token_id=VEND, tie_word_embeddings=False)
    else:
        cfg = transformers.Qwen3_5Config(text_config=dict(TEXT), vision_config=dict(VISION), image_token_id=IMG,
                                         video_token_id=VID, vision_start_token_id=VSTART, vision_end_token_id=VEND,
                                         tie_word_embeddings=False)
    cfg._attn_implementation = "eager"
    cfg.text_config._attn_implementation = "eager"
    cfg.vision_config._attn_implementation = "eager"
    torch.manual_seed(0)
    cls = transformers.Qwen3_5MoeForConditionalGeneration if moe else transformers.Qwen3_5ForConditionalGeneration
    model = cls(cfg).to(torch.float32)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "norm" in n or n.endswith("bias"):
                p.add_(torch.randn_like(p) * 0.1)
            if n.endswith("A_log"):
                p.uniform_(-1.0, 0.5)
    return model


def _save_hub_layout(model, path):
    """Write the checkpoint with the hub's tensor names (``model.visual.*``, ``model.language_model.*``)."""
    from safetensors.torch import save_file
    os.makedirs(path, exist_ok=True)
    save_file({k: v.detach().contiguous() for k, v in model.state_dict().items()},
              os.path.join(path, "model.safetensors"))
    cfg = model.config.to_dict()
    cfg["architectures"] = [type(model).__name__]
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    with open(os.path.join(path, "preprocessor_config.json"), "w") as f:
        json.dump({"patch_size": 4, "temporal_patch_size": 2, "merge_size": 2, "image_mean": [0.5, 0.5, 0.5],
                   "image_std": [0.5, 0.5, 0.5], "size": {"shortest_edge": 64, "longest_edge": 4096}}, f)


def test_image_preprocessing_matches_transformers():
    g = ImageGeometry(patch=4, temporal_patch=2, merge=2, min_pixels=64, max_pixels=4096)
    proc = transformers.Qwen2VLImageProcessor(patch_size=4, temporal_patch_size=2, merge_size=2,
                                              image_mean=[0.5] * 3, image_std=[0.5] * 3,
                                              size={"shortest_edge": 64, "longest_edge": 4096})
    torch.manual_seed(0)
    for H, W in [(32, 48), (24, 24), (50, 37), (90, 120)]:
        img = torch.randint(0, 256, (3, H, W), dtype=torch.uint8)
        want = proc(images=[img], return_tensors="pt")
        got = preprocess_frames([img], g)
        assert list(got.grid_thw) == want["image_grid_thw"][0].tolist(), (H, W)
        assert tuple(got.grid_thw[1:]) == tuple(s // 4 for s in smart_resize(H, W, 8, 64, 4096))
        # identical when no resize happens; within one 8-bit level of the torchvision bicubic otherwise
        tol = 1e-6 if (H % 8 == 0 and W % 8 == 0 and 64 <= H * W <= 4096) else 2.5 / 255 / 0.5
        assert float((got.pixel_values - want["pixel_values"]).abs().max()) <= tol, (H, W)


def test_vision_tower_matches_transformers():
    from transformers.models.qwen3_5.configuration_qwen3_5 import Qwen3_5VisionConfig
    from transformers.models.qwen3_5.modeling_qwen3_5 import Qwen3_5VisionModel
    vc = Qwen3_5VisionConfig(**VISION)
    vc._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = Qwen3_5VisionModel(vc).float().eval()
    with torch.no_grad():
        for p in hf.parameters():
            p.add_(torch.randn_like(p) * 0.05)
    vit = QwenVLViT(ViTConfig.from_hf(vc.to_dict()))
    vit.load_state(dict(hf.state_dict()))
    grids = [(1, 4, 6), (2, 8, 4), (1, 2, 2)]                  # two stills and a two-frame clip
    px = torch.randn(sum(t * h * w for t, h, w in grids), vit.cfg.patch_dim)
    with torch.no_grad():
        out = hf(px, torch.tensor(grids))
    mine, hidden = vit.encode(px, grids, return_hidden=True)
    assert float((hidden - out.last_hidden_state).norm() / out.last_hidden_state.norm()) < 1e-5
    assert float((mine - out.pooler_output).norm() / out.pooler_output.norm()) < 1e-5
    assert mine.shape == (sum(vit.rows_per_image(grids)), 64)


def _mm_sequence(seq_id, grids, seed, text_lens):
    """text, image, text, image, ..., text with random pixels; returns the Sequence."""
    g = torch.Generator().manual_seed(seed)
    segs = []
    for i, n in enumerate(text_lens):
        segs.append(torch.randint(0, 290, (n,), generator=g).tolist())
        if i < len(grids):
            t, h, w = grids[i]
            segs.append(ImageInputCPU(torch.randn(t * h * w, 3 * 2 * 4 * 4, generator=g), (t, h, w)))
    return build_multimodal_sequence(segs, IMG, merge=2, seq_id=seq_id, vision_start_token_id=VSTART,
                                     vision_end_token_id=VEND, train_on=[True] * len(segs))


def test_mrope_position_ids_match_transformers():
    model = _hf_vl_model()
    seq = _mm_sequence(0, [(1, 4, 6), (1, 8, 4)], 3, [5, 7, 9])
    ids = seq.tokens[None]
    types = (ids == IMG).to(torch.int32)
    want, _ = model.model.get_rope_index(ids, mm_token_type_ids=types,
                                         image_grid_thw=torch.tensor(seq.modality_inputs["grid_thw"]))
    got = compute_mrope_position_ids(seq, 0, len(seq))
    assert torch.equal(got.to(torch.int64).t(), want[:, 0])
    # a slice of the sequence (a chunk that starts inside the first image) sees the same positions
    assert torch.equal(compute_mrope_position_ids(seq, 9, 20), got[9:29])


def test_concat_splice_maps_and_gradients():
    a = _mm_sequence(0, [(1, 4, 4)], 1, [3, 2])                # 3 text, start, 4 placeholders, end, 2 text
    b = _mm_sequence(1, [], 2, [6])
    seqs = [a, b]
    # chunk 0: first 6 tokens of a (2 placeholders); chunk 1: rest of a, then b
    pieces = [[(0, 0, 6)], [(0, 6, len(a) - 6), (1, 0, 6)]]
    maps = build_splice_maps(seqs, pieces, [IMG], {0: 10})
    assert maps[0][0].tolist() == [4, 5] and maps[0][1].tolist() == [10, 11]
    assert maps[1][0].tolist() == [0, 1] and maps[1][1].tolist() == [12, 13]
    x = torch.zeros(6, 8)
    enc = torch.arange(14 * 8, dtype=torch.float32).view(14, 8)
    y = splice_forward(x, maps[0][0], enc[maps[0][1]])
    assert torch.equal(y[4], enc[10]) and torch.equal(y[5], enc[11]) and float(y[:4].abs().sum()) == 0
    dx = torch.ones(6, 8)
    dx, d_enc = splice_backward(dx, maps[0][0], want_encoder_grad=True)
    assert float(dx[4:].abs().sum()) == 0 and float(dx[:4].sum()) == 32 and d_enc.shape == (2, 8)


@pytest.mark.parametrize("chunk,moe", [(256, False), (32, False), (256, True)])
def test_vision_language_model_matches_transformers(tmp_path, chunk, moe):
    """Loss and text-side gradients of image + text sequences; ``chunk=32`` cuts sequences (and images) across
    chunks, so the rolling KV window, the recurrent state and the splice maps all cross chunk borders."""
    model = _hf_vl_model(moe)
    _save_hub_layout(model, str(tmp_path))
    seqs = [_mm_sequence(0, [(1, 4, 6), (1, 8, 4)], 3, [5, 7, 9]), _mm_sequence(1, [(1, 4, 4)], 4, [11, 6]),
            _mm_sequence(2, [], 5, [40])]
    # ---- transformers
    model.zero_grad()
    total = 0.0
    for s in seqs:
        ids = s.tokens[None]
        kw = {}
        if s.modality_inputs:
            kw = dict(pixel_values=s.modality_inputs["pixel_values"],
                      image_grid_thw=torch.tensor(s.modality_inputs["grid_thw"]),
                      mm_token_type_ids=(ids == IMG).to(torch.int32))
        logits = model(input_ids=ids, **kw).logits[0].float()
        total = total + torch.nn.functional.cross_entropy(logits, s.targets, ignore_index=-100, reduction="sum")
    total.backward()
    # ---- engine
    am = ft.from_pretrained(str(tmp_path), optimizer=ft.AdamW(lr=1e-3, state_dtype=torch.float32), max_seq_len=128,
                            max_global_batch_tokens=256, max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30,
                            device="cpu", compute_dtype=torch.float32, master_dtype=torch.float32,
                            grad_dtype=torch.float32, host_backend=UnpinnedHostBackend(), enable_multimodal=True,
                            working_set=ft.WorkingSetConfig.simple(max_seq_len=128, max_global_batch_tokens=256,
                                                                   chunk=chunk, round_tokens=256))
    assert am.embed.num_vision_layers() == 2
    st = am.fwd_bwd(seqs, loss_scale_factor=1.0)
    assert abs(st.loss_sum - float(total)) / float(total) < 2e-4, (st.loss_sum, float(total))
    assert am.embed.last_summary.n_images == 3 and am.embed.last_summary.n_image_tokens == 6 + 8 + 4
    sd = dict(model.named_parameters())
    g_embed = am.buffers.embed_grads()["g_tok_embeddings"]
    want = sd["model.language_model.embed_tokens.weight"].grad
    assert float((g_embed - want).norm() / want.norm()) < 2e-3
    assert float(g_embed[IMG].abs().max()) == 0.0              # placeholder rows never reach the embedding table
    g_head = am.buffers.head_grads()["g_head_proj"]
    assert float((g_head - sd["lm_head.weight"].grad).norm() / sd["lm_head.weight"].grad.norm()) < 2e-3
    g_o = am.buffers.grads(1)["g_o"]
    want = sd["model.language_model.layers.1.self_attn.o_proj.weight"].grad
    assert float((g_o - want).norm() / want.norm()) < 2e-3


def test_processor_bundle_reads_geometry_and_ids(tmp_path):
    model = _hf_vl_model()
    _save_hub_layout(model, str(tmp_path))
    b = MultimodalProcessorBundle.from_pretrained(str(tmp_path), load_tokenizer=False)
    assert (b.geometry.patch, b.geometry.temporal_patch, b.geometry.merge) == (4, 2, 2)
    assert (b.geometry.min_pixels, b.geometry.max_pixels) == (64, 4096)
    assert (b.image_token_id, b.vision_start_token_id, b.vision_end_token_id) == (IMG, VSTART, VEND)
    ims = b.process_images([torch.randint(0, 256, (3, 32, 48), dtype=torch.uint8)])
    assert ims[0].grid_thw == (1, 8, 12) and ims[0].pixel_values.shape == (96, 96)
    s = build_multimodal_sequence([[1, 2, 3], ims[0], [4, 5]], b.image_token_id, b.geometry.merge, 0,
                                  b.vision_start_token_id, b.vision_end_token_id, train_on=[False, False, True])
    assert len(s) == 3 + 1 + 24 + 1 + 2
    assert s.modality_inputs["image_spans"] == [(4, 1, 4, 6)]
    assert (s.targets != -100).sum() == 1 + 1                  # vision_end predicts 4, 4 predicts 5


def test_multimodal_training_follows_transformers_forward(tmp_path):
    """The engine owns the loop (vision tower frozen); before every step its current language-model weights are
    copied into the ``transformers`` model, which must give the same loss on the same batch.  The loss must also go
    down on the repeated batch (the reference's analogue: tests/test_qwen3_5_mm_train_parity.py)."""
    from flextrain_b200.io.hf_weights import collect_hf_state
    model = _hf_vl_model()
    _save_hub_layout(model, str(tmp_path))
    am = ft.from_pretrained(str(tmp_path), optimizer=ft.AdamW(lr=2e-3, state_dtype=torch.float32), max_seq_len=128,
                            max_global_batch_tokens=256, max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30,
                            device="cpu", compute_dtype=torch.float32, master_dtype=torch.float32,
                            grad_dtype=torch.float32, host_backend=UnpinnedHostBackend(), enable_multimodal=True,
                            working_set=ft.WorkingSetConfig.simple(max_seq_len=128, max_global_batch_tokens=256))
    seqs = [_mm_sequence(0, [(1, 4, 6)], 3, [5, 30]), _mm_sequence(1, [(1, 4, 4), (1, 2, 2)], 4, [8, 6, 20])]
    visual_before = {n: p.detach().clone() for n, p in model.named_parameters() if ".visual." in n}
    losses = []
    for step in range(4):
        state = collect_hf_state(am)                           # text-model names: model.layers..., lm_head.weight
        remap = {(k.replace("model.", "model.language_model.", 1) if k.startswith("model.") else k): v
                 for k, v in state.items()}
        missing = model.load_state_dict(remap, strict=False).missing_keys
        assert all(".visual." in k for k in missing), missing
        total = 0.0
        with torch.no_grad():
            for s in seqs:
                ids = s.tokens[None]
                logits = model(input_ids=ids, pixel_values=s.modality_inputs["pixel_values"],
                               image_grid_thw=torch.tensor(s.modality_inputs["grid_thw"]),
                               mm_token_type_ids=(ids == IMG).to(torch.int32)).logits[0].float()
                total += float(torch.nn.functional.cross_entropy(logits, s.targets, ignore_index=-100,
                                                                 reduction="sum"))
        st = am.fwd_bwd(seqs)
        am.step()
        assert abs(st.loss_sum - total) / total < 3e-4, (step, st.loss_sum, total)
        losses.append(st.loss)
    assert losses[-1] < losses[0] - 0.05, losses
    vit = am.embed.encoders["image"]
    for n, p in visual_before.items():                         # the frozen tower did not move
        mine = vit.w[n.split(".visual.", 1)[1]]
        assert torch.equal(mine.reshape(-1), p.reshape(-1)), n


def _chat_tokenizer(path):
    """Character-level tokenizer with vision special tokens and a chat template that renders image parts as
    ``<|vision_start|><|image_pad|><|vision_end|>`` (the shape of the Qwen-VL templates)."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    specials = ["<unk>", "</s>", "<|im_start|>", "<|im_end|>", "<|vision_start|>", "<|image_pad|>", "<|vision_end|>"]
    chars = specials + [chr(c) for c in range(32, 127)] + ["\n"]
    tok = Tokenizer(models.WordLevel({c: i for i, c in enumerate(chars)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Split("", behavior="isolated")
    tok.add_special_tokens(specials)
    fast = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", eos_token="</s>")
    fast.chat_template = (
        "{% for m in messages %}<|im_start|>{{ m['role'] }}\n"
        "{% if m['content'] is string %}{{ m['content'] }}{% else %}{% for p in m['content'] %}"
        "{% if p['type'] == 'image' %}<|vision_start|><|image_pad|><|vision_end|>{% else %}{{ p['text'] }}{% endif %}"
        "{% endfor %}{% endif %}<|im_end|>\n{% endfor %}"
        "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}")
    fast.save_pretrained(path)
    return fast, {s: fast.convert_tokens_to_ids(s) for s in specials}


def test_chat_rows_with_images_become_sequences(tmp_path):
    """Chat rows -> multimodal sequences through the tokenizer's template: every image part expands to its merged
    patch count between the template's vision tokens, MRoPE spans are recorded, and only the last answer is scored;
    the JSON source reads image files relative to the data file."""
    from PIL import Image
    import numpy as np
    d = str(tmp_path)
    fast, ids = _chat_tokenizer(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump({"image_token_id": ids["<|image_pad|>"], "vision_start_token_id": ids["<|vision_start|>"],
                   "vision_end_token_id": ids["<|vision_end|>"],
                   "vision_config": {"patch_size": 4, "temporal_patch_size": 2, "spatial_merge_size": 2}}, f)
    with open(os.path.join(d, "preprocessor_config.json"), "w") as f:
        json.dump({"patch_size": 4, "temporal_patch_size": 2, "merge_size": 2, "image_mean": [0.5] * 3,
                   "image_std": [0.5] * 3, "size": {"shortest_edge": 64, "longest_edge": 4096}}, f)
    b = MultimodalProcessorBundle.from_pretrained(d)
    assert b.tokenizer is not None and b.image_token_id == ids["<|image_pad|>"]
    rng = np.random.default_rng(0)
    Image.fromarray(rng.integers(0, 255, (32, 48, 3), dtype=np.uint8)).save(os.path.join(d, "a.png"))
    Image.fromarray(rng.integers(0, 255, (16, 16, 3), dtype=np.uint8)).save(os.path.join(d, "b.png"))
    msgs = [{"role": "user", "content": [{"type": "text", "text": "compare "}, {"type": "image"},
                                         {"type": "text", "text": " and "}, {"type": "image"}]},
            {"role": "assistant", "content": "first is wider"}]
    seq = b.build_from_messages(msgs, [Image.open(os.path.join(d, "a.png")), Image.open(os.path.join(d, "b.png"))])
    toks = seq.tokens.tolist()
    assert toks.count(ids["<|image_pad|>"]) == 4 * 6 + 2 * 2 and toks.count(ids["<|vision_start|>"]) == 2
    (s0, t0, h0, w0), (s1, t1, h1, w1) = seq.modality_inputs["image_spans"]
    assert (t0, h0, w0) == (1, 4, 6) and (t1, h1, w1) == (1, 2, 2)
    assert toks[s0 - 1] == ids["<|vision_start|>"] and toks[s0 + 24] == ids["<|vision_end|>"]
    assert toks[s1 - 1] == ids["<|vision_start|>"] and toks[s1 + 4] == ids["<|vision_end|>"]
    assert seq.modality_inputs["pixel_values"].shape == (8 * 12 + 4 * 4, 96)
    # scored targets are exactly the answer and what the template closes it with
    scored = [int(t) for t in seq.targets.tolist() if t != -100]
    answer = fast("first is wider", add_special_tokens=False)["input_ids"]
    assert scored[: len(answer)] == answer and len(scored) <= len(answer) + 2
    assert compute_mrope_position_ids(seq, 0, len(seq)).shape == (len(seq), 3)
    # the JSON source
    rows = [{"messages": msgs, "images": ["a.png", "b.png"]},
            {"messages": msgs, "images": ["missing.png", "b.png"]},                       # skipped: unreadable
            {"messages": [{"role": "user", "content": "no image here"}, {"role": "assistant", "content": "ok"}]}]
    with open(os.path.join(d, "mm.jsonl"), "w") as f:
        f.write("\n".join(json.dumps(r) for r in rows))
    src = ft.MultimodalJsonSource(os.path.join(d, "mm.jsonl"), b, max_seq_len=512, loop=False)
    got = list(src.iter_sequences())
    assert len(got) == 2 and src.skipped == 1 and got[1].modality_inputs is None
    assert torch.equal(got[0].tokens, seq.tokens)


def test_train_py_on_image_chat_rows(tmp_path):
    """``train.py --data-source mm_json`` end to end on CPU: a tiny vision-language checkpoint with its tokenizer and
    chat template, two chat rows with image files; the loss on the repeated rows goes down."""
    import re
    import subprocess
    import sys
    from PIL import Image
    import numpy as np
    d = str(tmp_path / "model")
    os.makedirs(d)
    fast, ids = _chat_tokenizer(d)
    cfg = transformers.Qwen3_5Config(text_config=dict(TEXT, vocab_size=len(fast)), vision_config=dict(VISION),
                                     image_token_id=ids["<|image_pad|>"], video_token_id=0,
                                     vision_start_token_id=ids["<|vision_start|>"],
                                     vision_end_token_id=ids["<|vision_end|>"], tie_word_embeddings=False)
    torch.manual_seed(0)
    _save_hub_layout(transformers.Qwen3_5ForConditionalGeneration(cfg).to(torch.float32), d)
    rng = np.random.default_rng(1)
    rows = []
    for i, (h, w) in enumerate([(32, 48), (16, 32)]):
        Image.fromarray(rng.integers(0, 255, (h, w, 3), dtype=np.uint8)).save(str(tmp_path / f"im{i}.png"))
        rows.append({"messages": [{"role": "user", "content": [{"type": "image"}, {"type": "text", "text": "what?"}]},
                                  {"role": "assistant", "content": f"picture number {i}"}], "images": [f"im{i}.png"]})
    with open(str(tmp_path / "rows.jsonl"), "w") as f:
        f.write("\n".join(json.dumps(r) for r in rows))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root + os.pathsep + os.environ.get("PYTHONPATH", ""), CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, os.path.join(root, "train.py"), "--model", d, "--mode", "full", "--data-source",
                        "mm_json", "--dataset", str(tmp_path / "rows.jsonl"), "--max-seq-len", "128",
                        "--max-global-batch-tokens", "256", "--steps", "8", "--lr", "5e-3", "--output-dir",
                        str(tmp_path / "run")], capture_output=True, text=True, env=env, timeout=900, cwd=str(tmp_path))
    assert r.returncode == 0, r.stderr[-3000:]
    losses = [float(m) for m in re.findall(r"\[step\s+\d+\].*? loss ([\d.]+)", r.stdout)]
    assert len(losses) == 8 and losses[-1] < losses[0] - 0.5, losses
