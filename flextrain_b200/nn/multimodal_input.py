"""Multimodal input layer (flextrain/nn/multimodal_input.py:83-355): token embedding + frozen modality encoders.

Once per round (:meth:`setup_round`) the images of the round's sequences are batched, copied to the device and
encoded under ``torch.inference_mode``; the host builds, per chunk, the map from placeholder rows to encoder rows.
Each chunk's embedded text then has its placeholder rows replaced by encoder rows (concat splice).  In backward the
placeholder rows of ``dx`` are zeroed before the embedding's scatter-add.  :meth:`finalize_round` drops the round's
encoder output."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..core.layer import ChunkMeta
from ..core.modality import ImageEmbeddings, ImageInputCPU, ImageInputs, InputsSummary
from .embed import TokenEmbedLayer
from .splices.concat import build_splice_maps, splice_backward, splice_forward


def images_of(seq) -> List[ImageInputCPU]:
    """The images a data adapter attached to a sequence, as :class:`ImageInputCPU` objects."""
    mi = seq.modality_inputs or {}
    if "images" in mi:
        return list(mi["images"])
    if "pixel_values" not in mi:
        return []
    out, off = [], 0
    for g in mi["grid_thw"]:
        n = int(g[0]) * int(g[1]) * int(g[2])
        out.append(ImageInputCPU(mi["pixel_values"][off:off + n], tuple(int(v) for v in g)))
        off += n
    return out


class MultimodalInputLayer:
    def __init__(self, text: TokenEmbedLayer, encoders: Dict[str, object], image_token_id: int,
                 video_token_id: Optional[int] = None):
        self.text = text
        self.encoders = encoders
        self.image_token_id = int(image_token_id)
        self.video_token_id = None if video_token_id is None else int(video_token_id)
        self.param_spec = text.param_spec
        self.vocab_size, self.d_model, self.scale = text.vocab_size, text.d_model, text.scale
        self._embeds: Optional[ImageEmbeddings] = None
        self.last_summary = InputsSummary()
        # a trainable tower: the round's encoder output with its graph, and the gradient that flows back into it
        self._rows_live: Optional[torch.Tensor] = None
        self._d_rows: Optional[torch.Tensor] = None
        self._opt_state: Dict[str, torch.Tensor] = {}
        self.encoder_prefix = "model.visual."                  # where the checkpoint keeps the tower's tensors
        self._reduced: Optional[Dict[str, torch.Tensor]] = None

    @property
    def placeholder_ids(self) -> List[int]:
        return [t for t in (self.image_token_id, self.video_token_id) if t is not None and t >= 0]

    def num_vision_layers(self) -> int:
        enc = self.encoders.get("image")
        return enc.cfg.depth if enc is not None else 0

    # ------------------------------------------------------------------ per round
    @property
    def train_encoders(self) -> bool:
        enc = self.encoders.get("image")
        return enc is not None and getattr(enc, "trainable", False)

    def setup_round(self, seqs, metas: List[ChunkMeta], device, train: bool = True) -> InputsSummary:
        """Encode every image of the round once and attach the splice maps to the chunks.  With a trainable tower
        and ``train`` the encoder's graph is kept until :meth:`finalize_round` sends the round's gradient through it."""
        enc = self.encoders.get("image")
        images, owner, row_offset, acc = [], [], {}, 0
        merge = enc.cfg.merge if enc is not None else 1
        for i, s in enumerate(seqs):
            ims = images_of(s)
            if not ims:
                continue
            if enc is None:
                raise RuntimeError("a sequence carries images but the model has no image encoder")
            row_offset[i] = acc
            for im in ims:
                im.validate(enc.cfg.patch_dim, merge)
                images.append(im)
                owner.append(i)
                acc += im.num_placeholders(merge)
        summary = InputsSummary(n_text_tokens=sum(len(s) for s in seqs) - acc, n_image_tokens=acc,
                                n_images=len(images), n_patches=sum(im.pixel_values.shape[0] for im in images))
        self.last_summary = summary
        self._embeds = None
        if not images:
            return summary
        batch = ImageInputs.pack(images, owner, enc.device, enc.dtype, pin=True)
        self._rows_live = self._d_rows = None
        if train and self.train_encoders:
            rows = enc.encode_train(batch.pixel_values, batch.grid_thw)
            self._rows_live = rows
            self._d_rows = torch.zeros(rows.shape, dtype=torch.float32, device=rows.device)
            rows = rows.detach()
        else:
            rows = enc.encode(batch.pixel_values, batch.grid_thw)
        self._embeds = ImageEmbeddings(rows.to(device), enc.rows_per_image(batch.grid_thw))
        maps = build_splice_maps(seqs, [m.extra["pieces"] for m in metas], self.placeholder_ids, row_offset)
        for i in row_offset:                                   # every image row must be consumed exactly once
            n_ph = int(torch.isin(seqs[i].tokens, torch.tensor(self.placeholder_ids)).sum())
            n_rows = sum(im.num_placeholders(merge) for im in images_of(seqs[i]))
            if n_ph != n_rows:
                raise ValueError(f"sequence {seqs[i].seq_id}: {n_ph} placeholder tokens but {n_rows} image rows")
        for m, mp in zip(metas, maps):
            if mp is not None:
                m.extra["mm_rows"] = mp[0].to(device, non_blocking=True)
                m.extra["mm_src"] = mp[1].to(device, non_blocking=True)
        return summary

    def finalize_round(self) -> None:
        if self._rows_live is not None:
            # every chunk of the round has handed its placeholder rows' gradient back: one backward through the tower
            self._rows_live.backward(self._d_rows.to(self._rows_live.dtype))
            self._reduced = None                               # the local gradient moved: any summed copy is stale
        self._rows_live = self._d_rows = None
        self._embeds = None

    # ------------------------------------------------------------------ trainable tower: gradients, update, state
    def encoder_grads(self) -> Dict[str, torch.Tensor]:
        """``{"g_" + name: fp32 gradient}`` of the tower's tensors (zeros where nothing has flowed yet)."""
        enc = self.encoders.get("image")
        if not self.train_encoders:
            return {}
        out = {}
        for n, m in enc.master.items():
            if m.grad is None:
                m.grad = torch.zeros_like(m)
            out["g_" + n] = m.grad
        return out

    def zero_encoder_grads(self) -> None:
        for g in self.encoder_grads().values():
            g.zero_()
        self._reduced = None

    def reduced_encoder_grads(self, process_group=None) -> Dict[str, torch.Tensor]:
        """The tower's gradient summed over the data-parallel ranks (a copy, made once per accumulated gradient: the
        local ``.grad`` tensors keep accumulating untouched, so a norm taken between two ``fwd_bwd`` calls does not
        disturb the sum).  Every rank calls it at the same points (``grad_norm`` / ``step``)."""
        local = self.encoder_grads()
        if process_group is None or not local:
            return local
        if getattr(self, "_reduced", None) is None:
            import torch.distributed as dist
            self._reduced = {k: g.clone() for k, g in local.items()}
            for k in sorted(self._reduced):                    # one fixed order on every rank
                dist.all_reduce(self._reduced[k], group=process_group)
        return self._reduced

    def step_encoders(self, optimizer, step_num: int, grad_scale: float = 1.0, process_group=None) -> int:
        """Update the tower with the engine's optimizer (state allocated on first use, fp32); the data-parallel ranks
        average nothing here: like every other gradient the tower's is a sum over the job's tokens."""
        enc = self.encoders.get("image")
        if not self.train_encoders:
            return 0
        grads = self.reduced_encoder_grads(process_group)
        spec = enc.param_spec()
        if not self._opt_state:
            for st in optimizer.state_specs(spec):
                self._opt_state[st.key] = torch.zeros(st.shape, dtype=st.dtype, device=enc.device)
        with torch.no_grad():
            rc = optimizer.step(spec, {n: m.data for n, m in enc.master.items()}, grads, self._opt_state, step_num,
                                grad_scale)
        enc.sync_compute()
        return int(rc or 0)

    def encoder_export_state(self) -> Dict[str, torch.Tensor]:
        """The tower's tensors under checkpoint names, for the exports (only when it trains: a frozen tower is passed
        through from the source directory)."""
        enc = self.encoders.get("image")
        if not self.train_encoders:
            return {}
        return {self.encoder_prefix + n: t for n, t in enc.export_state().items()}

    def encoder_state_dict(self) -> Dict[str, torch.Tensor]:
        """Masters and optimizer state of a trainable tower, for training-state checkpoints."""
        enc = self.encoders.get("image")
        if not self.train_encoders:
            return {}
        out = {"enc.master." + n: m.detach().cpu() for n, m in enc.master.items()}
        out.update({"enc.opt." + k: v.detach().cpu() for k, v in self._opt_state.items()})
        return out

    def load_encoder_state_dict(self, state: Dict[str, torch.Tensor]) -> None:
        enc = self.encoders.get("image")
        if not self.train_encoders:
            return
        with torch.no_grad():
            for n, m in enc.master.items():
                if "enc.master." + n in state:
                    m.copy_(state["enc.master." + n])
        self._opt_state = {k[len("enc.opt."):]: v.to(enc.device).clone() for k, v in state.items()
                           if k.startswith("enc.opt.")}
        enc.sync_compute()

    # ------------------------------------------------------------------ per chunk
    def forward(self, meta: ChunkMeta, params) -> torch.Tensor:
        x = self.text.forward(meta, params)
        rows = meta.extra.get("mm_rows")
        if rows is None:
            return x
        return splice_forward(x, rows, self._embeds.embeds.index_select(0, meta.extra["mm_src"]))

    def backward(self, dx, meta: ChunkMeta, params, grads) -> None:
        rows = meta.extra.get("mm_rows")
        if rows is not None:
            want = self._d_rows is not None
            dx, d_enc = splice_backward(dx, rows, want_encoder_grad=want)
            if want:
                self._d_rows.index_add_(0, meta.extra["mm_src"].to(self._d_rows.device),
                                        d_enc.to(self._d_rows.device, torch.float32))
        self.text.backward(dx, meta, params, grads)


def attach_multimodal_input(am, hf: dict, model_dir: str, freeze: bool = True, required: bool = False) -> None:
    """Swap the engine's token embedding for a :class:`MultimodalInputLayer` with the checkpoint's vision tower."""
    from ..io.hf_weights import SafetensorsDir
    from .encoders.qwen_vl_vit import QwenVLViT, ViTConfig
    vc = hf.get("vision_config")
    if not vc:
        if required:
            raise ValueError("enable_multimodal=True but config.json has no vision_config")
        return
    if am.tp is not None:
        raise NotImplementedError("multimodal input with tensor parallelism is not supported")
    vit = QwenVLViT(ViTConfig.from_hf(vc), device=am.device,
                    dtype=torch.bfloat16 if am.device.type == "cuda" else torch.float32)
    try:
        vit.load(SafetensorsDir(model_dir))
    except KeyError:
        if required:
            raise
        return
    if not freeze:
        if getattr(am, "dp", None) is not None and getattr(am.dp, "m", None) is not None:
            raise NotImplementedError("a trainable vision tower runs on one GPU or with FTB_DP_BACKEND=collective")
        vit.enable_training()
    am.embed = MultimodalInputLayer(am.embed, {"image": vit}, int(hf.get("image_token_id", -1)),
                                    hf.get("video_token_id"))
    am.embed.encoder_prefix = vit.loaded_prefix
