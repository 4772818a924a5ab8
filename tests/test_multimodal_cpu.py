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
    """Character-level tokenizer with vision special tokens and a chat template that renders image / video parts as
    ``<|vision_start|><|image_pad|><|vision_end|>`` / ``...<|video_pad|>...`` (the shape of the Qwen-VL templates)."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    specials = ["<unk>", "</s>", "<|im_start|>", "<|im_end|>", "<|vision_start|>", "<|image_pad|>", "<|vision_end|>",
                "<|video_pad|>"]
    chars = specials + [chr(c) for c in range(32, 127)] + ["\n"]
    tok = Tokenizer(models.WordLevel({c: i for i, c in enumerate(chars)}, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Split("", behavior="isolated")
    tok.add_special_tokens(specials)
    fast = transformers.PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", eos_token="</s>")
    fast.chat_template = (
        "{% for m in messages %}<|im_start|>{{ m['role'] }}\n"
        "{% if m['content'] is string %}{{ m['content'] }}{% else %}{% for p in m['content'] %}"
        "{% if p['type'] == 'image' %}<|vision_start|><|image_pad|><|vision_end|>"
        "{% elif p['type'] == 'video' %}<|vision_start|><|video_pad|><|vision_end|>{% else %}{{ p['text'] }}{% endif %}"
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
    # the reference's text form and its (pixel_values, grid) call
    from flextrain_b200.io.image_processing import preprocess_images
    text = fast.apply_chat_template(msgs, tokenize=False)
    seq_t = build_multimodal_sequence(text, [os.path.join(d, "a.png"), os.path.join(d, "b.png")], b)
    assert torch.equal(seq_t.tokens, seq.tokens)
    assert torch.equal(seq_t.modality_inputs["pixel_values"], seq.modality_inputs["pixel_values"])
    mask = torch.zeros(len(seq_t), dtype=torch.bool)
    mask[-5:] = True
    assert build_multimodal_sequence(text, [os.path.join(d, "a.png"), os.path.join(d, "b.png")], b,
                                     loss_mask=mask).active_token_count <= 5
    px, grid = preprocess_images([os.path.join(d, "a.png"), os.path.join(d, "b.png")], b)
    assert grid.tolist() == [[1, 8, 12], [1, 4, 4]] and torch.equal(px, seq.modality_inputs["pixel_values"])
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


# ---------------------------------------------------------------------------------------------------------- video

def test_video_preprocessing_matches_transformers():
    """Frame sampling, the clip's resize rule, patch order and the per-patch time stamps against the Qwen3-VL video
    processor / processor of ``transformers``."""
    import numpy as np
    from flextrain_b200.io.image_processing import sample_frame_indices, smart_resize_video, video_timestamps
    vp_cls = getattr(transformers, "Qwen3VLVideoProcessor", None)
    if vp_cls is None:
        pytest.skip("this transformers has no Qwen3VLVideoProcessor")
    from transformers.video_utils import VideoMetadata
    size = {"shortest_edge": 4 * 64, "longest_edge": 6 * 1024}
    proc = vp_cls(patch_size=4, temporal_patch_size=2, merge_size=2, image_mean=[0.5] * 3, image_std=[0.5] * 3,
                  size=size, do_sample_frames=False)
    g = ImageGeometry(patch=4, temporal_patch=2, merge=2, video_min_pixels=size["shortest_edge"],
                      video_max_pixels=size["longest_edge"])
    torch.manual_seed(0)
    for F, H, W in [(4, 32, 48), (5, 24, 24), (3, 50, 37), (8, 90, 120), (2, 8, 8)]:
        clip = torch.randint(0, 256, (F, 3, H, W), dtype=torch.uint8)
        want = proc(videos=[clip], return_tensors="pt")
        got = preprocess_frames(clip, g, video=True)
        assert got.kind == "video" and list(got.grid_thw) == want["video_grid_thw"][0].tolist(), (F, H, W)
        Hn, Wn = smart_resize_video(F, H, W, 2, 8, size["shortest_edge"], size["longest_edge"])
        assert tuple(got.grid_thw) == (-(-F // 2), Hn // 4, Wn // 4)
        tol = 1e-6 if (Hn, Wn) == (H, W) else 2.5 / 255 / 0.5
        assert float((got.pixel_values - want["pixel_values_videos"]).abs().max()) <= tol, (F, H, W)
    # which frames are kept
    for total, src_fps, fps in [(240, 24.0, 2.0), (30, 30.0, 2.0), (1000, 25.0, 1.0), (7, 24.0, 2.0), (100000, 30.0, 2.0)]:
        md = VideoMetadata(total_num_frames=total, fps=src_fps)
        want = proc.sample_frames(md, fps=fps).tolist()
        assert sample_frame_indices(total, src_fps, fps, proc.min_frames, proc.max_frames) == want, (total, src_fps)
    # what time each temporal patch shows
    from transformers.models.qwen3_vl.processing_qwen3_vl import Qwen3VLProcessor
    for idx, fps in [([0, 12, 24, 36], 24.0), ([0, 10, 20, 30, 40], 30.0), ([3], 25.0)]:
        want = Qwen3VLProcessor._calculate_timestamps(None, np.asarray(idx), fps, 2)
        assert video_timestamps(idx, fps, 2) == pytest.approx(want)


def _video_sequence(seq_id, seed):
    """text, a three-patch clip with a two-token time stamp before each patch, text, an image, text."""
    g = torch.Generator().manual_seed(seed)
    clip = ImageInputCPU(torch.randn(3 * 4 * 6, 3 * 2 * 4 * 4, generator=g), (3, 4, 6), kind="video",
                         frame_prefix_ids=[[200 + f, 210] for f in range(3)])
    img = ImageInputCPU(torch.randn(1 * 4 * 4, 3 * 2 * 4 * 4, generator=g), (1, 4, 4))
    text = lambda n: torch.randint(0, 200, (n,), generator=g).tolist()
    segs = [text(6), clip, text(5), img, text(9)]
    return build_multimodal_sequence(segs, IMG, merge=2, seq_id=seq_id, vision_start_token_id=VSTART,
                                     vision_end_token_id=VEND, train_on=[True] * len(segs), video_token_id=VID)


def test_video_sequence_layout_and_positions_match_transformers():
    model = _hf_vl_model()
    seq = _video_sequence(0, 11)
    ids = seq.tokens
    # three blocks of 2 x 3 merged patches, each after its two prefix tokens and between start / end tokens
    first = [int(i) for i in (ids == VID).nonzero().flatten()[::6]]
    assert int((ids == VID).sum()) == 18 and int((ids == IMG).sum()) == 4
    for f, p in enumerate(first):
        assert ids[p - 3:p].tolist() == [200 + f, 210, VSTART] and int(ids[p + 6]) == VEND
    # placeholders, wrappers and time stamps are never predicted
    assert not bool(torch.isin(seq.targets, torch.tensor([VID, IMG, VSTART, VEND, 200, 201, 202, 210])).any())
    assert int((seq.targets != -100).sum()) == (6 - 1) + 5 + 9      # every text token but the very first
    types = ((ids == IMG).to(torch.int32) + 2 * (ids == VID).to(torch.int32))[None]
    want, _ = model.model.get_rope_index(ids[None], mm_token_type_ids=types, image_grid_thw=torch.tensor([[1, 4, 4]]),
                                         video_grid_thw=torch.tensor([[3, 4, 6]]))
    got = compute_mrope_position_ids(seq, 0, len(seq))
    assert torch.equal(got.to(torch.int64).t(), want[:, 0])


@pytest.mark.parametrize("chunk", [256, 16])
def test_video_and_image_model_matches_transformers(tmp_path, chunk):
    """Loss and gradients of a sequence with a clip and an image; ``chunk=16`` cuts inside the clip's blocks."""
    model = _hf_vl_model()
    _save_hub_layout(model, str(tmp_path))
    seqs = [_video_sequence(0, 11), _mm_sequence(1, [(1, 4, 4)], 4, [11, 6])]
    model.zero_grad()
    total = 0.0
    for s in seqs:
        ids = s.tokens[None]
        ims = s.modality_inputs["images"]
        kw = dict(mm_token_type_ids=(ids == IMG).to(torch.int32) + 2 * (ids == VID).to(torch.int32))
        stills = [im for im in ims if im.kind == "image"]
        clips = [im for im in ims if im.kind == "video"]
        if stills:
            kw.update(pixel_values=torch.cat([im.pixel_values for im in stills]),
                      image_grid_thw=torch.tensor([im.grid_thw for im in stills]))
        if clips:
            kw.update(pixel_values_videos=torch.cat([im.pixel_values for im in clips]),
                      video_grid_thw=torch.tensor([im.grid_thw for im in clips]))
        logits = model(input_ids=ids, **kw).logits[0].float()
        total = total + torch.nn.functional.cross_entropy(logits, s.targets, ignore_index=-100, reduction="sum")
    total.backward()
    am = ft.from_pretrained(str(tmp_path), optimizer=ft.AdamW(lr=1e-3, state_dtype=torch.float32), max_seq_len=128,
                            max_global_batch_tokens=256, max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30,
                            device="cpu", compute_dtype=torch.float32, master_dtype=torch.float32,
                            grad_dtype=torch.float32, host_backend=UnpinnedHostBackend(), enable_multimodal=True,
                            working_set=ft.WorkingSetConfig.simple(max_seq_len=128, max_global_batch_tokens=256,
                                                                   chunk=chunk, round_tokens=256))
    st = am.fwd_bwd(seqs, loss_scale_factor=1.0)
    assert abs(st.loss_sum - float(total)) / float(total) < 2e-4, (st.loss_sum, float(total))
    assert am.embed.last_summary.n_images == 3 and am.embed.last_summary.n_image_tokens == 18 + 4 + 4
    sd = dict(model.named_parameters())
    g_embed = am.buffers.embed_grads()["g_tok_embeddings"]
    want = sd["model.language_model.embed_tokens.weight"].grad
    assert float((g_embed - want).norm() / want.norm()) < 2e-3
    assert float(g_embed[VID].abs().max()) == 0.0 and float(g_embed[IMG].abs().max()) == 0.0
    g_o = am.buffers.grads(1)["g_o"]
    want = sd["model.language_model.layers.1.self_attn.o_proj.weight"].grad
    assert float((g_o - want).norm() / want.norm()) < 2e-3


def test_chat_rows_with_videos_match_the_transformers_processor(tmp_path):
    """A chat row with a clip and an image: the token ids are what ``transformers``' Qwen3-VL processor makes of the
    same conversation (one ``<T seconds>`` + start + placeholders + end block per temporal patch); the JSON source
    reads clips from a ``.npy`` file, a frame directory and a frame list."""
    from PIL import Image
    import numpy as np
    vp_cls = getattr(transformers, "Qwen3VLVideoProcessor", None)
    if vp_cls is None:
        pytest.skip("this transformers has no Qwen3VLVideoProcessor")
    from transformers.video_utils import VideoMetadata
    d = str(tmp_path)
    fast, ids = _chat_tokenizer(d)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump({"image_token_id": ids["<|image_pad|>"], "video_token_id": ids["<|video_pad|>"],
                   "vision_start_token_id": ids["<|vision_start|>"], "vision_end_token_id": ids["<|vision_end|>"],
                   "vision_config": {"patch_size": 4, "temporal_patch_size": 2, "spatial_merge_size": 2}}, f)
    isize, vsize = {"shortest_edge": 64, "longest_edge": 4096}, {"shortest_edge": 256, "longest_edge": 8192}
    with open(os.path.join(d, "preprocessor_config.json"), "w") as f:
        json.dump({"patch_size": 4, "temporal_patch_size": 2, "merge_size": 2, "image_mean": [0.5] * 3,
                   "image_std": [0.5] * 3, "size": isize}, f)
    with open(os.path.join(d, "video_preprocessor_config.json"), "w") as f:
        json.dump({"size": vsize, "fps": 2, "min_frames": 4, "max_frames": 16}, f)
    b = MultimodalProcessorBundle.from_pretrained(d)
    assert b.video_token_id == ids["<|video_pad|>"] and b.geometry.video_max_pixels == 8192
    assert b.geometry.video_max_frames == 16
    rng = np.random.default_rng(0)
    recording = rng.integers(0, 255, (60, 24, 32, 3), dtype=np.uint8)            # 2.5 s at 24 frames per second
    still = Image.fromarray(rng.integers(0, 255, (16, 16, 3), dtype=np.uint8))
    msgs = [{"role": "user", "content": [{"type": "text", "text": "what happens in "}, {"type": "video"},
                                         {"type": "text", "text": " and in "}, {"type": "image"}]},
            {"role": "assistant", "content": "it moves"}]
    clip = b.process_video(torch.from_numpy(recording), source_fps=24.0)
    assert clip.grid_thw == (3, 6, 8) and len(clip.frame_prefix_ids) == 3       # 5 of 60 frames -> 3 temporal patches
    seq = b.build_from_messages(msgs, [still], videos=[clip])
    # ---- the same conversation through transformers
    ip = transformers.Qwen2VLImageProcessor(patch_size=4, temporal_patch_size=2, merge_size=2, image_mean=[0.5] * 3,
                                            image_std=[0.5] * 3, size=isize)
    vp = vp_cls(patch_size=4, temporal_patch_size=2, merge_size=2, image_mean=[0.5] * 3, image_std=[0.5] * 3,
                size=vsize, fps=2, min_frames=4, max_frames=16)
    proc = transformers.Qwen3VLProcessor(image_processor=ip, tokenizer=fast, video_processor=vp,
                                         chat_template=fast.chat_template)
    text = fast.apply_chat_template(msgs, tokenize=False, add_generation_prompt=False)
    want = proc(text=[text], images=[still], videos=[torch.from_numpy(recording).permute(0, 3, 1, 2)],
                video_metadata=[VideoMetadata(total_num_frames=60, fps=24.0)], return_tensors="pt")
    assert seq.tokens.tolist() == want["input_ids"][0].tolist()
    assert want["video_grid_thw"][0].tolist() == list(clip.grid_thw)
    assert float((clip.pixel_values - want["pixel_values_videos"]).abs().max()) <= 2.5 / 255 / 0.5
    rendered = fast.decode(seq.tokens.tolist()).replace(" ", "")               # the toy tokenizer spaces characters out
    assert "<0.3seconds>" in rendered and "<1.5seconds>" in rendered and rendered.count("seconds>") == 3
    scored = [int(t) for t in seq.targets.tolist() if t != -100]
    answer = fast("it moves", add_special_tokens=False)["input_ids"]
    assert scored[: len(answer)] == answer and len(scored) <= len(answer) + 2
    # ---- the JSON source: three ways to name a clip
    np.save(os.path.join(d, "rec.npy"), recording)
    still.save(os.path.join(d, "still.png"))
    os.makedirs(os.path.join(d, "frames"))
    kept = [0, 15, 30, 44, 59]
    for n, i in enumerate(kept):
        Image.fromarray(recording[i]).save(os.path.join(d, "frames", f"f{n:03d}.png"))
    rows = [{"messages": msgs, "images": ["still.png"], "videos": [{"path": "rec.npy", "fps": 24.0}]},
            {"messages": msgs, "images": ["still.png"],
             "videos": [{"path": "frames", "fps": 24.0, "frame_indices": kept}]},
            {"messages": msgs, "images": ["still.png"],
             "videos": [{"frames": [f"frames/f{n:03d}.png" for n in range(5)], "fps": 24.0, "frame_indices": kept}]},
            {"messages": msgs, "images": ["still.png"], "videos": []}]            # skipped: a video part without a clip
    with open(os.path.join(d, "mm.jsonl"), "w") as f:
        f.write("\n".join(json.dumps(r) for r in rows))
    src = ft.MultimodalJsonSource(os.path.join(d, "mm.jsonl"), b, max_seq_len=512, loop=False)
    got = list(src.iter_sequences())
    assert len(got) == 3 and src.skipped == 1
    for s in got:
        assert torch.equal(s.tokens, seq.tokens)
        assert torch.equal(s.modality_inputs["pixel_values"], seq.modality_inputs["pixel_values"])


def test_vision_language_export_reloads_in_transformers(tmp_path):
    """Fine-tune the text side of a vision-language checkpoint, export it, load the directory with ``transformers``
    as a vision-language model: the decoder comes back under the wrapper's own names with the trained values, the
    vision tower is passed through from the source, and the reloaded model's loss on image + text equals the
    engine's."""
    src_dir, out = str(tmp_path / "src"), str(tmp_path / "out")
    model = _hf_vl_model()
    _save_hub_layout(model, src_dir)
    am = ft.from_pretrained(src_dir, optimizer=ft.AdamW(lr=1e-2, state_dtype=torch.float32), max_seq_len=128,
                            max_global_batch_tokens=256, max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30,
                            device="cpu", compute_dtype=torch.float32, master_dtype=torch.float32,
                            grad_dtype=torch.float32, host_backend=UnpinnedHostBackend(), enable_multimodal=True)
    assert am.hf_nested_prefix == "model.language_model."
    seqs = [_mm_sequence(0, [(1, 4, 6)], 3, [5, 9]), _video_sequence(1, 11)]
    am.fwd_bwd(seqs, loss_scale_factor=1.0 / 64)
    am.step()
    ft.export.save_hf_full(am, out)
    re = transformers.AutoModelForImageTextToText.from_pretrained(out, dtype=torch.float32)
    re.config._attn_implementation = "eager"
    sd0, sd1 = model.state_dict(), re.state_dict()
    assert set(sd0) == set(sd1)
    for k in sd0:
        if ".visual." in k:
            assert torch.equal(sd0[k], sd1[k]), k                      # passed through unchanged
    moved = sd1["model.language_model.layers.1.self_attn.o_proj.weight"] - sd0["model.language_model.layers.1.self_attn.o_proj.weight"]
    assert float(moved.abs().max()) > 1e-3                             # the step is in the exported weights
    assert torch.allclose(sd1["model.language_model.layers.1.self_attn.o_proj.weight"], am.buffers.host_params(1)["w_o"])
    want = 0.0
    with torch.no_grad():
        for s in seqs:
            ids = s.tokens[None]
            ims = s.modality_inputs["images"]
            kw = dict(mm_token_type_ids=(ids == IMG).to(torch.int32) + 2 * (ids == VID).to(torch.int32))
            stills = [im for im in ims if im.kind == "image"]
            clips = [im for im in ims if im.kind == "video"]
            if stills:
                kw.update(pixel_values=torch.cat([im.pixel_values for im in stills]),
                          image_grid_thw=torch.tensor([im.grid_thw for im in stills]))
            if clips:
                kw.update(pixel_values_videos=torch.cat([im.pixel_values for im in clips]),
                          video_grid_thw=torch.tensor([im.grid_thw for im in clips]))
            logits = re(input_ids=ids, **kw).logits[0].float()
            want += float(torch.nn.functional.cross_entropy(logits, s.targets, ignore_index=-100, reduction="sum"))
    got = am.evaluate(seqs)
    assert abs(got.loss_sum - want) / want < 2e-4, (got.loss_sum, want)


def test_vision_language_lora_adapter_names_the_wrapper_modules(tmp_path):
    """The adapter of a vision-language checkpoint addresses the decoder where the wrapper class holds it
    (``model.language_model.layers``); applied to the ``transformers`` model by the PEFT rule it gives the engine's
    loss on image + text."""
    from safetensors import safe_open
    src_dir, ad = str(tmp_path / "src"), str(tmp_path / "adapter")
    model = _hf_vl_model()
    _save_hub_layout(model, src_dir)
    f32 = torch.float32
    am = ft.from_pretrained(src_dir, optimizer=ft.AdamW(lr=1e-2, state_dtype=f32), max_seq_len=128,
                            max_global_batch_tokens=256, max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30,
                            device="cpu", compute_dtype=f32, master_dtype=f32, grad_dtype=f32,
                            host_backend=UnpinnedHostBackend(), enable_multimodal=True, lora_targets="all",
                            lora_rank=4, lora_alpha=8.0, lora_adapter_compute_dtype=f32,
                            lora_adapter_master_dtype=f32, lora_adapter_grad_dtype=f32,
                            lora_adapter_opt_state_dtype=f32)
    torch.manual_seed(3)
    for _, _, n, t in am.named_master_params():
        if n.endswith("_lora_b"):
            t.copy_(torch.randn_like(t) * 0.3)
    seqs = [_mm_sequence(0, [(1, 4, 6)], 3, [5, 9])]
    want = am.evaluate(seqs).loss_sum
    ft.export.save_lora_adapter(am, ad)
    scale = 8.0 / 4
    sd = dict(model.named_parameters())
    applied = 0
    with safe_open(os.path.join(ad, "adapter_model.safetensors"), framework="pt") as f, torch.no_grad():
        for k in f.keys():
            assert k.startswith("base_model.model.model.language_model.layers."), k
            if k.endswith("lora_A.weight"):
                mod = k[len("base_model.model."): -len(".lora_A.weight")]
                sd[mod + ".weight"].add_(scale * (f.get_tensor(k.replace("lora_A", "lora_B")) @ f.get_tensor(k)))
                applied += 1
    assert applied >= 7
    s = seqs[0]
    ids = s.tokens[None]
    with torch.no_grad():
        logits = model(input_ids=ids, pixel_values=s.modality_inputs["pixel_values"],
                       image_grid_thw=torch.tensor(s.modality_inputs["grid_thw"]),
                       mm_token_type_ids=(ids == IMG).to(torch.int32)).logits[0].float()
    got = float(torch.nn.functional.cross_entropy(logits, s.targets, ignore_index=-100, reduction="sum"))
    assert abs(got - want) / want < 2e-4, (got, want)


def test_trainable_vision_tower_matches_transformers(tmp_path):
    """``freeze_modality_encoders=False``: the gradient that reaches the placeholder rows flows on through the tower
    (one backward per round, images and a clip, sequences cut across chunks); the tower's gradients equal
    ``transformers``' autograd, an optimizer step moves it, the export carries the new tower and an exact-resume
    checkpoint restores it."""
    src_dir, out = str(tmp_path / "src"), str(tmp_path / "out")
    model = _hf_vl_model()
    _save_hub_layout(model, src_dir)
    build = lambda: ft.from_pretrained(
        src_dir, optimizer=ft.AdamW(lr=1e-2, state_dtype=torch.float32), max_seq_len=128, max_global_batch_tokens=256,
        max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30, device="cpu", compute_dtype=torch.float32,
        master_dtype=torch.float32, grad_dtype=torch.float32, host_backend=UnpinnedHostBackend(), enable_multimodal=True,
        freeze_modality_encoders=False,
        working_set=ft.WorkingSetConfig.simple(max_seq_len=128, max_global_batch_tokens=256, chunk=32, round_tokens=128))
    am = build()
    assert am.embed.train_encoders
    seqs = [_mm_sequence(0, [(1, 4, 6), (1, 8, 4)], 3, [5, 7, 9]), _video_sequence(1, 11), _mm_sequence(2, [], 5, [40])]
    model.zero_grad()
    total = 0.0
    for s in seqs:
        ids = s.tokens[None]
        kw = dict(mm_token_type_ids=(ids == IMG).to(torch.int32) + 2 * (ids == VID).to(torch.int32)) if s.modality_inputs else {}
        ims = (s.modality_inputs or {}).get("images", [])
        stills, clips = [im for im in ims if im.kind == "image"], [im for im in ims if im.kind == "video"]
        if stills:
            kw.update(pixel_values=torch.cat([im.pixel_values for im in stills]),
                      image_grid_thw=torch.tensor([im.grid_thw for im in stills]))
        if clips:
            kw.update(pixel_values_videos=torch.cat([im.pixel_values for im in clips]),
                      video_grid_thw=torch.tensor([im.grid_thw for im in clips]))
        logits = model(input_ids=ids, **kw).logits[0].float()
        total = total + torch.nn.functional.cross_entropy(logits, s.targets, ignore_index=-100, reduction="sum")
    total.backward()
    st = am.fwd_bwd(seqs, loss_scale_factor=1.0)               # two rounds: the tower's gradient accumulates over them
    assert st.n_rounds >= 2 and abs(st.loss_sum - float(total)) / float(total) < 2e-4
    sd = dict(model.named_parameters())
    grads = am.embed.encoder_grads()
    checked = 0
    for n, g in grads.items():
        want = sd["model.visual." + n[2:]].grad
        want = want.reshape(g.shape)
        assert float((g - want).norm()) <= 2e-3 * float(want.norm()) + 1e-7, n
        checked += 1
    assert checked == len(am.embed.encoders["image"].w) and checked > 20
    before = {n: t.clone() for n, t in am.embed.encoders["image"].w.items()}
    gn = am.grad_norm()
    assert gn > float(torch.sqrt(sum(g.pow(2).sum() for g in grads.values())))      # the tower is part of the norm
    assert am.step() == 0
    moved = [n for n, t in am.embed.encoders["image"].w.items() if not torch.equal(t, before[n])]
    assert len(moved) == len(before)
    loss1 = am.evaluate(seqs).loss_sum
    assert loss1 < st.loss_sum
    # export: the trained tower, in the checkpoint's shapes; reload in transformers gives the engine's loss
    ft.export.save_hf_full(am, out)
    re = transformers.AutoModelForImageTextToText.from_pretrained(out, dtype=torch.float32)
    rsd = re.state_dict()
    assert rsd["model.visual.patch_embed.proj.weight"].shape == model.state_dict()["model.visual.patch_embed.proj.weight"].shape
    assert not torch.equal(rsd["model.visual.blocks.0.attn.qkv.weight"], model.state_dict()["model.visual.blocks.0.attn.qkv.weight"])
    assert torch.allclose(rsd["model.visual.blocks.0.attn.qkv.weight"], am.embed.encoders["image"].w["blocks.0.attn.qkv.weight"])
    from safetensors import safe_open
    with safe_open(am.save_hf(str(tmp_path / "single"), out_filename="w.safetensors"), framework="pt") as f:
        assert torch.allclose(f.get_tensor("model.visual.blocks.0.attn.qkv.weight"),
                              am.embed.encoders["image"].w["blocks.0.attn.qkv.weight"])
    # exact resume: tower masters and optimizer state travel with the training state
    am.save_training_state(str(tmp_path / "state"))
    am.fwd_bwd(seqs, loss_scale_factor=1.0)
    am.step()
    want_w = {n: t.clone() for n, t in am.embed.encoders["image"].w.items()}
    bm = build()
    bm.load_training_state(str(tmp_path / "state"))
    bm.fwd_bwd(seqs, loss_scale_factor=1.0)
    bm.step()
    for n, t in bm.embed.encoders["image"].w.items():
        assert torch.equal(t, want_w[n]), n
    # a frozen tower stays put and the evaluation path keeps no graph
    fz = ft.from_pretrained(src_dir, optimizer=ft.AdamW(lr=1e-2), max_seq_len=128, max_global_batch_tokens=256,
                            max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30, device="cpu",
                            compute_dtype=torch.float32, master_dtype=torch.float32, grad_dtype=torch.float32,
                            host_backend=UnpinnedHostBackend(), enable_multimodal=True)
    assert not fz.embed.train_encoders and fz.embed.encoder_grads() == {}
    am.evaluate(seqs)
    assert am.embed._rows_live is None


def _tower_rank(rank, world, port, src_dir, out):
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        am = ft.from_pretrained(src_dir, optimizer=ft.AdamW(lr=1e-2, state_dtype=torch.float32), max_seq_len=128,
                                max_global_batch_tokens=256, max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30,
                                device="cpu", compute_dtype=torch.float32, master_dtype=torch.float32,
                                grad_dtype=torch.float32, host_backend=UnpinnedHostBackend(), enable_multimodal=True,
                                freeze_modality_encoders=False, world_size=world, rank=rank)
        seqs = _tower_batch()
        am.fwd_bwd(seqs[rank::world], loss_scale_factor=1.0 / 64)
        norm = am.grad_norm()
        assert am.step(max_grad_norm=0.5 * norm) == 0
        w = am.embed.encoders["image"].w
        out.put((rank, norm, {n: t.numpy() for n, t in w.items()}))
    finally:
        dist.destroy_process_group()


def _tower_batch():
    return [_mm_sequence(0, [(1, 4, 6)], 3, [5, 9]), _video_sequence(1, 11), _mm_sequence(2, [(1, 4, 4)], 4, [11, 6]),
            _mm_sequence(3, [], 5, [40])]


def test_trainable_vision_tower_on_two_data_parallel_ranks(tmp_path):
    """Two CPU ranks, each with half of the sequences: the tower's gradient is summed over the ranks before the norm
    and the update, so norm and updated tower equal the single-process run on all sequences."""
    import socket
    import torch.multiprocessing as mp
    src_dir = str(tmp_path / "src")
    _save_hub_layout(_hf_vl_model(), src_dir)
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_tower_rank, args=(r, 2, port, src_dir, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=600) for _ in range(2)], key=lambda x: x[0])
    for p in procs:
        p.join(60)
    am = ft.from_pretrained(src_dir, optimizer=ft.AdamW(lr=1e-2, state_dtype=torch.float32), max_seq_len=128,
                            max_global_batch_tokens=256, max_gpu_mem_bytes=8 << 30, max_host_mem_bytes=8 << 30,
                            device="cpu", compute_dtype=torch.float32, master_dtype=torch.float32,
                            grad_dtype=torch.float32, host_backend=UnpinnedHostBackend(), enable_multimodal=True,
                            freeze_modality_encoders=False)
    am.fwd_bwd(_tower_batch(), loss_scale_factor=1.0 / 64)
    norm = am.grad_norm()
    assert am.step(max_grad_norm=0.5 * norm) == 0
    assert abs(res[0][1] - norm) < 1e-4 * norm and abs(res[1][1] - norm) < 1e-4 * norm
    for n, t in am.embed.encoders["image"].w.items():
        for r in range(2):
            # AdamW's first step is sign-like: an element whose gradient is at rounding level may move the other way,
            # so compare in the mean and bound the share of elements that differ
            d = (torch.from_numpy(res[r][2][n]) - t).abs()
            assert float(d.mean()) < 2e-4 and float((d > 1e-3).float().mean()) < 0.02, (r, n, float(d.mean()))
    assert all((res[0][2][n] == res[1][2][n]).all() for n in res[0][2])            # the ranks stay identical
