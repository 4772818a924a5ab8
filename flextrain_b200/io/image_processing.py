"""Image pre-processing for multimodal SFT (flextrain/io/image_processing.py:40-278).

The reference wraps HuggingFace's ``AutoImageProcessor``; here the Qwen-VL family's pre-processing is written out in
torch (so a training job needs neither PIL nor the processor classes on its hot path) and is checked against
``transformers``' ``Qwen2VLImageProcessor`` in the tests:

1. *smart resize*: both sides become multiples of ``patch * merge``, the area is kept inside
   ``[min_pixels, max_pixels]`` and the aspect ratio is preserved as well as that allows (bicubic, anti-aliased,
   rounded back to 8-bit levels as an 8-bit image pipeline does);
2. rescale to ``[0, 1]`` and normalise per channel;
3. a still image is repeated to fill the temporal patch; frames of a video are grouped ``temporal_patch`` at a time;
4. the result is cut into ``temporal_patch x patch x patch`` blocks, flattened channel-major, and ordered
   merge-block-major: the ``merge x merge`` patches that the vision tower's merger concatenates are consecutive rows.

Video clips go the same way with three differences, each checked against ``transformers``' Qwen3-VL video processor:
frames are sampled at a target rate (:func:`sample_frame_indices`), the pixel budget of the resize counts all frames
(:func:`smart_resize_video`), and in the text every temporal patch is a block of its own, ``<T seconds>`` + vision
start + its placeholders + vision end, with ``T`` the mean time of the frames in the patch (:func:`video_timestamps`).

:class:`MultimodalProcessorBundle` reads the geometry and the special token ids from a model directory
(``preprocessor_config.json`` / ``video_preprocessor_config.json`` / ``config.json``) and, when a tokenizer is there,
turns chat-style rows with images and videos into multimodal :class:`Sequence` objects;
:func:`build_multimodal_sequence` does the token-level assembly."""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, List, Optional, Sequence as Seq, Tuple

import torch

from ..core.modality import ImageInputCPU
from .sequence import Sequence

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(height: int, width: int, factor: int, min_pixels: int, max_pixels: int) -> Tuple[int, int]:
    """Target size: multiples of ``factor``, area within ``[min_pixels, max_pixels]``, aspect ratio kept."""
    if max(height, width) / max(min(height, width), 1) > 200:
        raise ValueError(f"aspect ratio of a {height}x{width} image is beyond 200")
    h = round(height / factor) * factor
    w = round(width / factor) * factor
    if h * w > max_pixels:
        beta = math.sqrt(height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return max(h, factor), max(w, factor)


def smart_resize_video(num_frames: int, height: int, width: int, temporal_factor: int, factor: int,
                       min_pixels: int, max_pixels: int) -> Tuple[int, int]:
    """Frame size of a clip: multiples of ``factor``, with frames x height x width inside the pixel budget."""
    if height < factor or width < factor:
        raise ValueError(f"a {height}x{width} frame is smaller than patch*merge = {factor}")
    if max(height, width) / min(height, width) > 200:
        raise ValueError(f"aspect ratio of a {height}x{width} frame is beyond 200")
    h = round(height / factor) * factor
    w = round(width / factor) * factor
    t = math.ceil(num_frames / temporal_factor) * temporal_factor
    if t * h * w > max_pixels:
        beta = math.sqrt(num_frames * height * width / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif t * h * w < min_pixels:
        beta = math.sqrt(min_pixels / (num_frames * height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def sample_frame_indices(total_frames: int, source_fps: float, target_fps: float = 2.0, min_frames: int = 4,
                         max_frames: int = 768) -> List[int]:
    """Which frames of a ``total_frames``-long clip recorded at ``source_fps`` to keep for ``target_fps`` frames per
    second: evenly spaced, at least ``min_frames`` and at most ``max_frames`` (and never more than there are)."""
    n = int(total_frames / source_fps * target_fps)
    n = min(max(n, min_frames), max_frames, total_frames)
    if n <= 1:
        return [0] * max(n, 1)
    step = (total_frames - 1) / (n - 1)
    # round half to even, as numpy's rint does
    return [int(round(i * step)) for i in range(n)]


def video_timestamps(frame_indices: Seq[int], source_fps: float, temporal_patch: int = 2) -> List[float]:
    """Seconds shown in front of each temporal patch: the mean of its first and last frame's time."""
    idx = [int(i) for i in frame_indices]
    if len(idx) % temporal_patch:
        idx += [idx[-1]] * (temporal_patch - len(idx) % temporal_patch)
    ts = [i / source_fps for i in idx]
    return [(ts[i] + ts[i + temporal_patch - 1]) / 2 for i in range(0, len(ts), temporal_patch)]


def _to_uint8_chw(img: Any) -> torch.Tensor:
    """PIL image, ``(H, W, 3)`` uint8 array, or ``(3, H, W)`` tensor (uint8, or float in [0, 1]) -> ``(3, H, W)`` float
    tensor holding 8-bit levels."""
    if isinstance(img, torch.Tensor):
        t = img
        if t.dim() == 3 and t.shape[0] not in (1, 3) and t.shape[-1] in (1, 3):
            t = t.permute(2, 0, 1)
        t = t.to(torch.float32) * (255.0 if t.dtype.is_floating_point else 1.0)
    else:
        import numpy as np
        if hasattr(img, "convert"):                    # PIL
            img = img.convert("RGB")
        a = np.asarray(img)
        if a.ndim == 2:
            a = a[:, :, None].repeat(3, axis=2)
        t = torch.from_numpy(a.copy()).permute(2, 0, 1).to(torch.float32)
    if t.shape[0] == 1:
        t = t.expand(3, -1, -1)
    return t


@dataclass
class ImageGeometry:
    patch: int = 16
    temporal_patch: int = 2
    merge: int = 2
    min_pixels: int = 64 * 64
    max_pixels: int = 16 * 16 * 4 * 4096
    mean: Tuple[float, float, float] = (0.5, 0.5, 0.5)
    std: Tuple[float, float, float] = (0.5, 0.5, 0.5)
    # video clips: pixel budget over all frames of a clip, and the frame sampling rule
    video_min_pixels: int = 128 * 32 * 32
    video_max_pixels: int = 768 * 32 * 32
    video_fps: float = 2.0
    video_min_frames: int = 4
    video_max_frames: int = 768

    @property
    def patch_dim(self) -> int:
        return 3 * self.temporal_patch * self.patch * self.patch


def preprocess_frames(frames: Seq[Any], g: ImageGeometry, resize: bool = True,
                      video: Optional[bool] = None) -> ImageInputCPU:
    """One image (a single frame) or one video clip (several frames of equal size) -> :class:`ImageInputCPU`.
    ``video`` (default: more than one frame) selects the clip's resize rule and marks the result as a clip."""
    if isinstance(frames, torch.Tensor) and frames.dim() == 4:                 # (F, H, W, 3) or (F, 3, H, W)
        frames = list(frames)
    ts = [_to_uint8_chw(f) for f in frames]
    video = len(ts) > 1 if video is None else bool(video)
    H, W = ts[0].shape[-2:]
    if any(t.shape[-2:] != (H, W) for t in ts):
        raise ValueError("the frames of a clip must have one size")
    x = torch.stack(ts, 0)                                                     # (F, 3, H, W), 8-bit levels
    q = g.patch * g.merge
    if resize:
        if video:
            Hn, Wn = smart_resize_video(len(ts), H, W, g.temporal_patch, q, g.video_min_pixels, g.video_max_pixels)
        else:
            Hn, Wn = smart_resize(H, W, q, g.min_pixels, g.max_pixels)
        if (Hn, Wn) != (H, W):
            # on 8-bit data, as an image library does it (the two separable passes each saturate to 8 bits)
            x8 = x.round().clamp_(0, 255).to(torch.uint8)
            x = torch.nn.functional.interpolate(x8, size=(Hn, Wn), mode="bicubic", align_corners=False,
                                                antialias=True).to(torch.float32)
            H, W = Hn, Wn
    elif H % q or W % q:
        raise ValueError(f"a {H}x{W} image is not a multiple of patch*merge = {q}; pass resize=True")
    mean, std = torch.tensor(g.mean).view(1, 3, 1, 1), torch.tensor(g.std).view(1, 3, 1, 1)
    x = (x / 255.0 - mean) / std
    tp = g.temporal_patch
    if x.shape[0] % tp:
        x = torch.cat([x, x[-1:].expand(tp - x.shape[0] % tp, -1, -1, -1)], 0)
    gt, gh, gw = x.shape[0] // tp, H // g.patch, W // g.patch
    m, p = g.merge, g.patch
    x = x.view(gt, tp, 3, gh // m, m, p, gw // m, m, p)
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(gt * gh * gw, 3 * tp * p * p)
    return ImageInputCPU(pixel_values=x.contiguous(), grid_thw=(gt, gh, gw), kind="video" if video else "image")


def _open_images(images: Seq[Any]) -> List[Any]:
    out = []
    for im in images:
        if isinstance(im, (str, os.PathLike)):
            from PIL import Image
            im = Image.open(im).convert("RGB")
        out.append(im)
    return out


def preprocess_images(images: Seq[Any], g: Any = None, resize: bool = True):
    """Images (objects or paths) -> one :class:`ImageInputCPU` each.  Given a :class:`MultimodalProcessorBundle` in
    place of the geometry (the reference's call, flextrain/io/image_processing.py:112-143) the result is the pair
    ``(pixel_values, image_grid_thw)`` of all images instead."""
    if hasattr(g, "geometry"):
        ims = [preprocess_frames([im], g.geometry, resize=resize) for im in _open_images(images)]
        return (torch.cat([im.pixel_values for im in ims], 0) if ims else torch.empty(0, g.geometry.patch_dim),
                torch.tensor([list(im.grid_thw) for im in ims], dtype=torch.int64).reshape(-1, 3))
    g = g or ImageGeometry()
    return [preprocess_frames([im], g, resize=resize) for im in _open_images(images)]


def patchify(img: torch.Tensor, patch: int = 16, temporal_patch: int = 2, merge: int = 2) -> ImageInputCPU:
    """``img (3, H, W)`` float in [0, 1] with the default geometry otherwise; kept for callers of the first API."""
    return preprocess_frames([img], ImageGeometry(patch=patch, temporal_patch=temporal_patch, merge=merge))


def build_multimodal_sequence(segments: Seq[Any], image_token_id: int, merge: int = 2, seq_id: int = 0,
                              vision_start_token_id: Optional[int] = None, vision_end_token_id: Optional[int] = None,
                              train_on: Optional[Seq[bool]] = None, video_token_id: Optional[int] = None,
                              video_start_token_id: Optional[int] = None,
                              video_end_token_id: Optional[int] = None, targets: Optional[torch.Tensor] = None,
                              loss_mask: Optional[torch.Tensor] = None) -> Sequence:
    """Assemble token ids, images and video clips into one training sequence.

    ``segments`` alternates freely between lists of token ids and :class:`ImageInputCPU` objects; every image expands
    to ``[vision_start] + image_token * n + [vision_end]`` with ``n`` its merged patch count.  A clip
    (``kind == "video"``) expands to one such block per temporal patch, made of ``video_token_id`` and wrapped in
    ``video_start_token_id`` / ``video_end_token_id`` (default: the image's start / end ids), each preceded by the
    clip's ``frame_prefix_ids`` entry (the ``<T seconds>`` text) when it has one; for the rotary positions every
    block is a single-frame image.  ``train_on[i]`` says whether the tokens of text segment ``i`` (counting all
    segments) are targets; placeholder and wrapper tokens never are, and the token before one never predicts it."""
    if isinstance(segments, str):             # the reference's call: (text, images, bundle, *, targets, loss_mask)
        return build_multimodal_sequence_from_text(segments, image_token_id, merge, targets=targets, loss_mask=loss_mask)
    if targets is not None or loss_mask is not None:
        raise TypeError("targets / loss_mask belong to the text form; with segments use train_on")
    ids: List[int] = []
    learn: List[bool] = []
    images: List[ImageInputCPU] = []
    spans = []
    v_start = vision_start_token_id if video_start_token_id is None else video_start_token_id
    v_end = vision_end_token_id if video_end_token_id is None else video_end_token_id

    def block(start_id, token, n, end_id, gh, gw):
        if start_id is not None:
            ids.append(start_id); learn.append(False)
        first = len(ids)
        spans.append((first, 1, gh // merge, gw // merge))
        ids.extend([token] * n)
        learn.extend([False] * n)
        if end_id is not None:
            ids.append(end_id); learn.append(False)
        return first

    for si, seg in enumerate(segments):
        if isinstance(seg, ImageInputCPU):
            t, gh, gw = seg.grid_thw
            per_frame = (gh // merge) * (gw // merge)
            if seg.kind == "video":
                if video_token_id is None:
                    raise ValueError("a video clip needs video_token_id")
                pre = seg.frame_prefix_ids
                if pre is not None and len(pre) != t:
                    raise ValueError(f"{len(pre)} frame prefixes for {t} temporal patches")
                for f in range(t):
                    if pre is not None:
                        ids.extend(int(v) for v in pre[f]); learn.extend([False] * len(pre[f]))
                    first = block(v_start, video_token_id, per_frame, v_end, gh, gw)
                    if f == 0:
                        seg.first_token = first
            else:
                if t != 1:                                     # a multi-frame "image": one block, t advances inside it
                    if vision_start_token_id is not None:
                        ids.append(vision_start_token_id); learn.append(False)
                    seg.first_token = len(ids)
                    spans.append((len(ids), t, gh // merge, gw // merge))
                    ids.extend([image_token_id] * (t * per_frame)); learn.extend([False] * (t * per_frame))
                    if vision_end_token_id is not None:
                        ids.append(vision_end_token_id); learn.append(False)
                else:
                    seg.first_token = block(vision_start_token_id, image_token_id, per_frame, vision_end_token_id, gh, gw)
            images.append(seg)
        else:
            seg = [int(v) for v in seg]
            ids += seg
            learn += [True if train_on is None else bool(train_on[si])] * len(seg)
    toks = torch.tensor(ids, dtype=torch.int64)
    tgt = torch.roll(toks, -1)
    tgt[-1] = -100
    keep = torch.tensor(learn[1:] + [False])                 # position i predicts token i + 1
    tgt[~keep] = -100
    mi = None
    if images:
        mi = {"pixel_values": torch.cat([im.pixel_values for im in images], 0),
              "grid_thw": [tuple(im.grid_thw) for im in images], "image_spans": spans, "images": images}
    return Sequence(toks, targets=tgt, seq_id=seq_id, modality_inputs=mi)


def build_multimodal_sequence_from_text(text: str, images: Seq[Any], bundle: "MultimodalProcessorBundle", *,
                                        targets: Optional[torch.Tensor] = None,
                                        loss_mask: Optional[torch.Tensor] = None) -> Sequence:
    """The reference's text form (flextrain/io/image_processing.py:146-278): ``text`` is the rendered conversation
    with ONE image placeholder per image (and the vision start / end markers around it); every placeholder is expanded
    to its image's merged patch count.  ``targets`` / ``loss_mask``, when given, are for the expanded sequence;
    by default every text token is a target and placeholders are not."""
    if bundle.tokenizer is None:
        raise RuntimeError("this model directory has no tokenizer; use build_multimodal_sequence with token ids")
    ids = bundle._flat_ids(bundle.tokenizer(text, add_special_tokens=False))
    ims = [preprocess_frames([im], bundle.geometry) for im in _open_images(images)]
    if sum(1 for t in ids if t == bundle.image_token_id) != len(ims):
        raise ValueError(f"the text has {sum(1 for t in ids if t == bundle.image_token_id)} image placeholders for "
                         f"{len(ims)} images")
    segs: List[Any] = []
    cur: List[int] = []
    k = 0
    for t in ids:
        if t == bundle.image_token_id:
            if cur:
                segs.append(cur)
            segs.append(ims[k])
            k, cur = k + 1, []
        else:
            cur.append(t)
    if cur:
        segs.append(cur)
    seq = build_multimodal_sequence(segs, bundle.image_token_id, bundle.geometry.merge)
    if targets is not None:
        if len(targets) != len(seq):
            raise ValueError(f"targets has {len(targets)} entries for {len(seq)} tokens")
        seq.targets = torch.as_tensor(targets).to(torch.int64)
    if loss_mask is not None:
        if len(loss_mask) != len(seq):
            raise ValueError(f"loss_mask has {len(loss_mask)} entries for {len(seq)} tokens")
        seq.loss_mask = torch.as_tensor(loss_mask)
    return seq


@dataclass
class MultimodalProcessorBundle:
    """Geometry + special token ids of one model directory, and its tokenizer when ``transformers`` can load one."""
    model_path: str
    geometry: ImageGeometry
    image_token_id: int
    vision_start_token_id: Optional[int] = None
    vision_end_token_id: Optional[int] = None
    video_token_id: Optional[int] = None
    tokenizer: Any = None
    image_placeholder: str = "<|image_pad|>"
    extra: dict = field(default_factory=dict)

    @classmethod
    def from_pretrained(cls, model_path: str, load_tokenizer: bool = True) -> "MultimodalProcessorBundle":
        with open(os.path.join(model_path, "config.json")) as f:
            cfg = json.load(f)
        vc = cfg.get("vision_config") or {}
        g = ImageGeometry(patch=int(vc.get("patch_size", 16)), temporal_patch=int(vc.get("temporal_patch_size", 2)),
                          merge=int(vc.get("spatial_merge_size", 2)))
        pp = os.path.join(model_path, "preprocessor_config.json")
        if os.path.exists(pp):
            with open(pp) as f:
                pc = json.load(f)
            g.patch = int(pc.get("patch_size", g.patch))
            g.temporal_patch = int(pc.get("temporal_patch_size", g.temporal_patch))
            g.merge = int(pc.get("merge_size", g.merge))
            size = pc.get("size") or {}
            g.min_pixels = int(pc.get("min_pixels", size.get("shortest_edge", g.min_pixels)))
            g.max_pixels = int(pc.get("max_pixels", size.get("longest_edge", g.max_pixels)))
            if pc.get("image_mean"):
                g.mean = tuple(float(v) for v in pc["image_mean"])
            if pc.get("image_std"):
                g.std = tuple(float(v) for v in pc["image_std"])
        vp = os.path.join(model_path, "video_preprocessor_config.json")
        if os.path.exists(vp):
            with open(vp) as f:
                vpc = json.load(f)
            size = vpc.get("size") or {}
            g.video_min_pixels = int(size.get("shortest_edge", g.video_min_pixels))
            g.video_max_pixels = int(size.get("longest_edge", g.video_max_pixels))
            g.video_fps = float(vpc.get("fps") or g.video_fps)
            g.video_min_frames = int(vpc.get("min_frames", g.video_min_frames))
            g.video_max_frames = int(vpc.get("max_frames", g.video_max_frames))
        tok = None
        if load_tokenizer:
            try:
                from transformers import AutoTokenizer
                tok = AutoTokenizer.from_pretrained(model_path)
            except Exception:                                  # no tokenizer files: token-id level API only
                tok = None
        return cls(model_path=model_path, geometry=g, image_token_id=int(cfg.get("image_token_id", -1)),
                   vision_start_token_id=cfg.get("vision_start_token_id"),
                   vision_end_token_id=cfg.get("vision_end_token_id"), video_token_id=cfg.get("video_token_id"),
                   tokenizer=tok)

    def process_images(self, images: Seq[Any]) -> List[ImageInputCPU]:
        return preprocess_images(images, self.geometry)

    def process_video(self, frames: Seq[Any], source_fps: Optional[float] = None,
                      frame_indices: Optional[Seq[int]] = None, sample: bool = True) -> ImageInputCPU:
        """One clip -> :class:`ImageInputCPU` of kind ``"video"`` with its ``<T seconds>`` prefixes.

        ``frames`` are the clip's frames in order (a ``(F, H, W, 3)`` / ``(F, 3, H, W)`` array or a list of images).
        With ``source_fps`` and ``sample=True`` they are the whole recording and are thinned to the geometry's target
        rate; otherwise they are taken as already sampled, ``frame_indices`` saying which frames of the recording
        they were (default: consecutive, at 24 frames per second when ``source_fps`` is not given either)."""
        n = len(frames)
        g = self.geometry
        if frame_indices is None:
            if sample and source_fps is not None:
                frame_indices = sample_frame_indices(n, source_fps, g.video_fps, g.video_min_frames, g.video_max_frames)
                frames = [frames[i] for i in frame_indices]
            else:
                frame_indices = list(range(n))
        elif len(frame_indices) != n:
            raise ValueError(f"{len(frame_indices)} frame indices for {n} frames")
        clip = preprocess_frames(frames, g, video=True)
        if self.tokenizer is not None:
            stamps = video_timestamps(frame_indices, source_fps or 24.0, g.temporal_patch)
            clip.frame_prefix_ids = [self.tokenizer(f"<{t:.1f} seconds>", add_special_tokens=False)["input_ids"]
                                     for t in stamps]
        return clip

    def build(self, texts: Seq[str], images: Seq[Any], seq_id: int = 0, train_on: Optional[Seq[bool]] = None) -> Sequence:
        """``texts`` has one more entry than ``images``: text, image, text, image, ..., text.  ``train_on`` flags the
        text pieces (default: only the last one, the answer)."""
        if self.tokenizer is None:
            raise RuntimeError("this model directory has no tokenizer; use build_multimodal_sequence with token ids")
        if len(texts) != len(images) + 1:
            raise ValueError("need len(texts) == len(images) + 1")
        # an entry that is already an ImageInputCPU (a clip from process_video, say) is used as it is
        ims = [im if isinstance(im, ImageInputCPU) else preprocess_frames([im], self.geometry) for im in images]
        segs: List[Any] = []
        flags: List[bool] = []
        for i, t in enumerate(texts):
            segs.append(self.tokenizer(t, add_special_tokens=False)["input_ids"])
            flags.append((i == len(texts) - 1) if train_on is None else bool(train_on[i]))
            if i < len(ims):
                segs.append(ims[i])
                flags.append(False)
        return build_multimodal_sequence(segs, self.image_token_id, self.geometry.merge, seq_id,
                                         self.vision_start_token_id, self.vision_end_token_id, flags,
                                         video_token_id=self.video_token_id)

    def build_from_messages(self, messages: Seq[dict], images: Seq[Any], seq_id: int = 0,
                            max_seq_len: Optional[int] = None, videos: Seq[Any] = ()) -> Optional[Sequence]:
        """Chat-style row -> multimodal sequence, through the tokenizer's own chat template.

        ``messages`` is the usual list of ``{"role", "content"}`` dicts whose ``content`` is a string or a list of
        ``{"type": "text", "text": ...}`` / ``{"type": "image"}`` / ``{"type": "video"}`` parts; the template must
        render every image part as one image placeholder token, which is expanded here to the image's merged patch
        count, and every video part as one video placeholder token (between vision start / end tokens or bare), which
        is replaced by the clip's per-temporal-patch blocks.  ``videos`` are clips from :meth:`process_video` or
        frame lists (taken as already sampled).  Only the LAST assistant message is trained on (everything the
        template renders before it is prompt).  Returns ``None`` when ``max_seq_len`` is given and the result is
        longer."""
        if self.tokenizer is None or not hasattr(self.tokenizer, "apply_chat_template"):
            raise RuntimeError("this model directory has no tokenizer with a chat template")
        if not messages or messages[-1].get("role") != "assistant":
            raise ValueError("the last message must be the assistant's answer")
        ids_of = lambda msgs, gen: self._flat_ids(self.tokenizer.apply_chat_template(msgs, tokenize=True,
                                                                                    add_generation_prompt=gen))
        full, prompt = ids_of(list(messages), False), ids_of(list(messages[:-1]), True)
        if full[: len(prompt)] != prompt:
            raise ValueError("the chat template does not render the prompt as a prefix of the whole conversation")
        ims = self.process_images(images)
        n_ph = sum(1 for t in full if t == self.image_token_id)
        if n_ph != len(ims):
            raise ValueError(f"the template rendered {n_ph} image placeholders for {len(ims)} images")
        clips = [v if isinstance(v, ImageInputCPU) else self.process_video(v, sample=False) for v in videos]
        n_vp = sum(1 for t in full if t == self.video_token_id) if self.video_token_id is not None else 0
        if n_vp != len(clips):
            raise ValueError(f"the template rendered {n_vp} video placeholders for {len(clips)} videos")
        segs: List[Any] = []
        flags: List[bool] = []
        cur: List[int] = []
        cur_start, k, kv, skip = 0, 0, 0, -1
        for pos, t in enumerate(full):
            if pos == skip:                                    # the vision end token the template wrote after a video
                cur_start = pos + 1
                continue
            if clips and t == self.video_token_id:
                # every temporal patch gets its own start / end tokens: drop the pair the template wrote around
                # the single placeholder
                if cur and self.vision_start_token_id is not None and cur[-1] == self.vision_start_token_id:
                    cur.pop()
                if (self.vision_end_token_id is not None and pos + 1 < len(full)
                        and full[pos + 1] == self.vision_end_token_id):
                    skip = pos + 1
                if cur:
                    segs.append(cur); flags.append(cur_start >= len(prompt))
                segs.append(clips[kv]); flags.append(False)
                kv += 1
                cur, cur_start = [], pos + 1
            elif t == self.image_token_id:
                if cur:
                    segs.append(cur); flags.append(cur_start >= len(prompt))
                segs.append(ims[k]); flags.append(False)
                k += 1
                cur, cur_start = [], pos + 1
            else:
                if cur and (cur_start < len(prompt)) != (pos < len(prompt)):      # prompt / answer border
                    segs.append(cur); flags.append(cur_start >= len(prompt))
                    cur, cur_start = [], pos
                if not cur:
                    cur_start = pos
                cur.append(int(t))
        if cur:
            segs.append(cur); flags.append(cur_start >= len(prompt))
        # the template already wrote the vision start / end tokens around each placeholder
        seq = build_multimodal_sequence(segs, self.image_token_id, self.geometry.merge, seq_id, None, None, flags,
                                        video_token_id=self.video_token_id,
                                        video_start_token_id=self.vision_start_token_id,
                                        video_end_token_id=self.vision_end_token_id)
        if max_seq_len is not None and len(seq) > max_seq_len:
            return None
        return seq

    @staticmethod
    def _flat_ids(out) -> List[int]:
        if isinstance(out, dict) or hasattr(out, "input_ids"):
            out = out["input_ids"]
        if out and isinstance(out[0], (list, tuple)):
            out = out[0]
        return [int(t) for t in out]
