"""Token sources (flextrain/io/sources.py:84-1245).

``TokenSource`` protocol: ``get_sequences(max_token_count)`` returns whole sequences whose total
length does not exceed the budget, ``iter_sequences()`` streams them, ``push_back(seqs)`` returns
unconsumed sequences to the front of the queue (used by the short-tail-round spill in train.py).
Adapters: synthetic uniform tokens, raw token lists, FineWeb-style ``uint16`` ``.bin`` shards, JSON /
JSONL SFT records (background tokenizer thread, prompt masking), custom-schema records, and a
streaming HuggingFace ``datasets`` adapter.
"""
from __future__ import annotations

import collections
import glob
import itertools
import json
import os
import queue
import threading
from typing import Callable, Deque, Iterable, Iterator, List, Optional, Protocol, Sequence as Seq

import numpy as np
import torch

from .sequence import Sequence

IGNORE = -100


class TokenSource(Protocol):
    def get_sequences(self, max_token_count: int) -> List[Sequence]: ...
    def iter_sequences(self) -> Iterator[Sequence]: ...
    def push_back(self, seqs: Seq[Sequence]) -> None: ...


class _QueueMixin:
    """Front queue shared by all sources: pushed-back sequences are served first, in order."""

    def _init_queue(self):
        self._front: Deque[Sequence] = collections.deque()

    def push_back(self, seqs: Seq[Sequence]) -> None:
        for s in reversed(list(seqs)):
            self._front.appendleft(s)

    def _next(self) -> Optional[Sequence]:
        if self._front:
            return self._front.popleft()
        try:
            return next(self._it)
        except StopIteration:
            return None

    def get_sequences(self, max_token_count: int) -> List[Sequence]:
        out, total = [], 0
        while True:
            s = self._next()
            if s is None:
                break
            if total + len(s) > max_token_count:
                if not out and len(s) > max_token_count:
                    raise ValueError(f"sequence of {len(s)} tokens exceeds the step budget {max_token_count}")
                self._front.appendleft(s)
                break
            out.append(s)
            total += len(s)
        return out

    def iter_sequences(self) -> Iterator[Sequence]:
        while True:
            s = self._next()
            if s is None:
                return
            yield s


class RankStridedSource(_QueueMixin):
    """Data-parallel view of a source: rank ``r`` of ``n`` sees sequences ``r, r + n, r + 2n, ...`` of the wrapped
    source, so ranks that read the same files train on disjoint data."""

    def __init__(self, source, rank: int, world: int):
        if not 0 <= rank < world:
            raise ValueError(f"rank {rank} outside world {world}")
        self.source, self.rank, self.world = source, rank, world
        self._init_queue()
        self._it = itertools.islice(source.iter_sequences(), rank, None, world)


class MultimodalJsonSource(_QueueMixin):
    """JSON / JSONL rows ``{"messages": [...], "images": [path, ...], "videos": [clip, ...]}`` (chat parts of type
    ``image`` / ``video`` mark where each goes) -> multimodal sequences through a
    :class:`MultimodalProcessorBundle`; paths are relative to the file.  A clip is a ``.npy`` file holding
    ``(frames, H, W, 3)`` 8-bit pixels, a directory of frame images (read in name order), a list of frame image
    paths, or ``{"path" | "frames": one of those, "fps": rate of the recording, "frame_indices": [...],
    "sample": bool}``: with ``fps`` and no ``frame_indices`` the frames are the whole recording and are thinned to
    the model's rate unless ``sample`` is false.  Rows that fail to load or exceed ``max_seq_len`` are skipped and
    counted in ``skipped``."""
    FRAME_SUFFIXES = (".png", ".jpg", ".jpeg", ".bmp", ".webp")

    def __init__(self, path: str, bundle, max_seq_len: int, loop: bool = True):
        self.path, self.bundle, self.max_seq_len, self.loop = path, bundle, max_seq_len, loop
        with open(path) as f:
            txt = f.read().strip()
        self.records = json.loads(txt) if txt.startswith("[") else [json.loads(l) for l in txt.splitlines() if l.strip()]
        self.skipped = 0
        self._init_queue()
        self._it = self._generate()

    def _clip(self, spec, base: str):
        from PIL import Image
        opts = spec if isinstance(spec, dict) else {}
        src = (opts.get("path") or opts.get("frames")) if isinstance(spec, dict) else spec
        if src is None:
            raise ValueError("a video entry needs 'path' or 'frames'")
        full = lambda p: p if os.path.isabs(p) else os.path.join(base, p)
        if isinstance(src, str) and src.endswith(".npy"):
            frames = list(torch.from_numpy(np.load(full(src))))
        else:
            if isinstance(src, str):
                d = full(src)
                src = [os.path.join(d, n) for n in sorted(os.listdir(d)) if n.lower().endswith(self.FRAME_SUFFIXES)]
            frames = [Image.open(full(p)).convert("RGB") for p in src]
        if not frames:
            raise ValueError("a video entry has no frames")
        return self.bundle.process_video(frames, source_fps=opts.get("fps"), frame_indices=opts.get("frame_indices"),
                                         sample=bool(opts.get("sample", True)))

    def _generate(self) -> Iterator[Sequence]:
        from PIL import Image
        base, sid = os.path.dirname(os.path.abspath(self.path)), 0
        while True:
            emitted = 0
            for r in self.records:
                try:
                    ims = [Image.open(p if os.path.isabs(p) else os.path.join(base, p)).convert("RGB")
                           for p in r.get("images", [])]
                    clips = [self._clip(v, base) for v in r.get("videos", [])]
                    seq = self.bundle.build_from_messages(r["messages"], ims, seq_id=sid, max_seq_len=self.max_seq_len,
                                                          videos=clips)
                except (OSError, ValueError, KeyError):
                    seq = None
                if seq is None:
                    self.skipped += 1
                    continue
                sid += 1
                emitted += 1
                yield seq
            if not self.loop or emitted == 0:
                return


class SyntheticTokenSource(_QueueMixin):
    """Uniform random tokens from a seed; fixed length or a cycle of lengths; infinite
    (flextrain/io/sources.py:795-853). ``targets = roll(tokens, -1)``."""

    def __init__(self, vocab_size: int, seq_len=None, seed: int = 0, pin: bool = False, *, seq_lens=None):
        self.vocab_size = vocab_size
        seq_len = seq_lens if seq_len is None else seq_len        # ``seq_lens`` is the reference's spelling
        seq_len = 512 if seq_len is None else seq_len
        self.lengths = [int(seq_len)] if isinstance(seq_len, int) else [int(x) for x in seq_len]
        if not self.lengths:
            raise ValueError("seq_lens must be non-empty")
        self.gen = torch.Generator().manual_seed(seed)
        self.pin = pin
        self._count = 0
        self._init_queue()
        self._it = self._generate()

    def _generate(self) -> Iterator[Sequence]:
        while True:
            n = self.lengths[self._count % len(self.lengths)]
            toks = torch.randint(0, self.vocab_size, (n,), generator=self.gen, dtype=torch.int64)
            if self.pin and torch.cuda.is_available():
                toks = toks.pin_memory()
            yield Sequence(toks, seq_id=self._count)
            self._count += 1


class RawTokenSource(_QueueMixin):
    """Pre-tokenised sequences supplied by the caller (flextrain/io/sources.py:137-209): a list of 1-D id tensors /
    lists, a list of ``{"tokens", "targets"?, "loss_mask"?}`` dicts, or one dict of such lists."""

    def __init__(self, tokens: Iterable, loop: bool = False):
        ent = []
        if isinstance(tokens, dict):
            n = len(tokens["tokens"])
            for i in range(n):
                ent.append((tokens["tokens"][i], (tokens.get("targets") or [None] * n)[i],
                            (tokens.get("loss_mask") or [None] * n)[i]))
        else:
            for item in tokens:
                if isinstance(item, dict):
                    ent.append((item["tokens"], item.get("targets"), item.get("loss_mask")))
                else:
                    ent.append((item, None, None))
        as64 = lambda t: None if t is None else torch.as_tensor(t).to(torch.int64)
        self._data = [(as64(t), as64(g), None if m is None else torch.as_tensor(m)) for t, g, m in ent]
        self.loop = loop
        self.reset()

    def reset(self) -> None:
        self._init_queue()
        self._it = self._generate()

    def _generate(self):
        i = 0
        while True:
            for t, g, m in self._data:
                yield Sequence(t.clone(), targets=None if g is None else g.clone(), loss_mask=m, seq_id=i)
                i += 1
            if not self.loop or not self._data:
                return


class ShardTokenSource(_QueueMixin):
    """FineWeb-style shards: ``uint16`` token files, optionally with a 256-int32 header (magic 20240520)
    (flextrain/io/sources.py:861-1012).  Two ways to cut them:

    * ``seq_len`` given: fixed windows of ``seq_len`` tokens with next-token targets (pre-training on a packed stream);
    * ``max_seq_len`` given instead: one sequence per document, documents being what lies between ``end_id`` tokens
      (a leading ``start_id`` is dropped), shorter than ``min_seq_len`` skipped, longer than ``max_seq_len`` truncated,
      ids clipped to ``vocab_size``.

    ``pattern`` is a path, a glob, a list of paths, or a ``{shard_index:06d}`` format string numbered from 1 to
    ``num_shards``; ``num_shards`` also limits a glob."""
    MAGIC = 20240520

    def __init__(self, pattern=None, seq_len: Optional[int] = None, loop: bool = True, vocab_size: Optional[int] = None,
                 *, num_shards: Optional[int] = None, min_seq_len: int = 32, max_seq_len: Optional[int] = None,
                 shard_pattern: Optional[str] = None, token_dtype=None, start_id: int = 50256, end_id: int = 50256):
        pattern = shard_pattern if pattern is None else pattern
        if pattern is None:
            raise ValueError("ShardTokenSource needs a shard pattern")
        if isinstance(pattern, (list, tuple)):                 # explicit shard list, kept in the given order
            self.files = [str(p) for p in pattern]
        elif "{shard_index" in pattern:
            if num_shards is None:
                raise ValueError("num_shards is needed with a {shard_index} pattern")
            self.files = [pattern.format(shard_index=i) for i in range(1, num_shards + 1)]
        else:
            self.files = sorted(glob.glob(pattern)) if any(c in pattern for c in "*?[") else [pattern]
        if num_shards is not None:
            self.files = self.files[:num_shards]
        if not self.files:
            raise FileNotFoundError(f"no shard matches {pattern!r}")
        if seq_len is None and max_seq_len is None:
            raise ValueError("give seq_len (fixed windows) or max_seq_len (one sequence per document)")
        self.seq_len, self.loop, self.vocab_size = seq_len, loop, vocab_size
        self.min_seq_len, self.max_seq_len = int(min_seq_len), max_seq_len
        self.token_dtype = np.dtype(token_dtype or np.uint16)
        self.start_id, self.end_id = int(start_id), int(end_id)
        self.reset()

    def reset(self) -> None:
        self._init_queue()
        self._it = self._generate() if self.seq_len is not None else self._documents()

    def _read(self, path: str) -> np.ndarray:
        with open(path, "rb") as f:
            head = np.frombuffer(f.read(1024), dtype=np.int32)
        if head.size == 256 and head[0] == self.MAGIC:
            return np.memmap(path, dtype=self.token_dtype, mode="r", offset=1024)
        return np.memmap(path, dtype=self.token_dtype, mode="r")

    def _generate(self):
        sid = 0
        while True:
            for path in self.files:
                arr = self._read(path)
                for a in range(0, len(arr) - self.seq_len - 1, self.seq_len):
                    win = torch.from_numpy(np.asarray(arr[a:a + self.seq_len + 1], dtype=np.int64))
                    yield Sequence(win[:-1].clone(), targets=win[1:].clone(), seq_id=sid)
                    sid += 1
            if not self.loop:
                return

    def _documents(self):
        sid = 0
        while True:
            emitted = 0
            for path in self.files:
                arr = self._read(path)
                ends = np.flatnonzero(np.asarray(arr) == self.end_id).tolist() + [len(arr)]
                a = 0
                for e in ends:
                    raw = arr[a:e]
                    a = e + 1
                    if len(raw) and int(raw[0]) == self.start_id:
                        raw = raw[1:]
                    if len(raw) < max(self.min_seq_len, 1):
                        continue
                    doc = np.asarray(raw[: self.max_seq_len], dtype=np.int64)
                    if self.vocab_size:
                        doc = np.clip(doc, 0, self.vocab_size - 1)
                    yield Sequence(torch.from_numpy(doc.copy()), seq_id=sid)
                    sid += 1
                    emitted += 1
            if not self.loop or emitted == 0:
                return


PROMPT_TEMPLATE = "Instruction:\n{instruction}\n\nResponse:\n"


from .download import normalise_sft_record  # noqa: E402  (pure Python; lives where login-node tools can load it)


class JsonSFTTokenSource(_QueueMixin):
    """JSON / JSONL SFT records tokenised by a background thread; loss only on response tokens
    (flextrain/io/sources.py:238-790).  Generic wrapper
    ``"Instruction:\\n{instruction}\\n\\nResponse:\\n{response}<EOS>"`` with ``add_special_tokens=False``, or the
    tokenizer's own chat template with ``apply_chat_template=True``.  Records longer than ``max_seq_len`` are
    dropped, or have their response truncated with ``truncate_long=True``."""

    def __init__(self, path: str, tokenizer, max_seq_len: int = 2048, *, apply_chat_template: bool = False,
                 truncate_long: bool = False, loop: bool = True, prefetch: int = 256, shuffle_seed: Optional[int] = None,
                 prompt_field: str = "instruction", response_field: str = "output", input_field: Optional[str] = "input",
                 min_seq_len: int = 0, trust_remote_code: bool = False, prefetch_max_tokens: Optional[int] = None):
        if isinstance(tokenizer, str):                         # a model directory / hub id, as the reference accepts
            from transformers import AutoTokenizer
            tokenizer = AutoTokenizer.from_pretrained(tokenizer, trust_remote_code=trust_remote_code)
        self.path, self.tok, self.max_seq_len = path, tokenizer, max_seq_len
        self.chat, self.truncate, self.loop = apply_chat_template, truncate_long, loop
        self.prompt_field, self.response_field, self.input_field = prompt_field, response_field, input_field
        self.min_seq_len = int(min_seq_len)
        if prefetch_max_tokens is not None:                    # the reference bounds its look-ahead in tokens
            prefetch = max(1, min(prefetch, int(prefetch_max_tokens) // max(int(max_seq_len), 1)))
        self.records = self._load(path)
        if shuffle_seed is not None:
            rng = np.random.default_rng(shuffle_seed)
            rng.shuffle(self.records)
        self.dropped = 0
        self._q: "queue.Queue" = queue.Queue(maxsize=prefetch)
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._producer, daemon=True)
        self._thread.start()
        self._init_queue()
        self._it = self._consume()

    @staticmethod
    def _load(path: str) -> List[dict]:
        with open(path) as f:
            txt = f.read().strip()
        if txt.startswith("["):
            return json.loads(txt)
        return [json.loads(line) for line in txt.splitlines() if line.strip()]

    def _fields(self, rec: dict) -> Optional[dict]:
        """The record as ``{"instruction", "response"}``: the configured field names first, then the usual schemas."""
        pf, rf = getattr(self, "prompt_field", None), getattr(self, "response_field", None)
        if pf and rf and pf in rec and rf in rec and (pf, rf) != ("instruction", "output"):
            ins = str(rec[pf])
            extra = getattr(self, "input_field", None)
            if extra and rec.get(extra):
                ins = f"{ins}\n{rec[extra]}"
            return {"instruction": ins, "response": str(rec[rf])}
        return normalise_sft_record(rec)

    def encode(self, rec: dict) -> Optional[Sequence]:
        r = self._fields(rec)
        if r is None:
            return None
        eos = getattr(self.tok, "eos_token_id", None)
        if self.chat and hasattr(self.tok, "apply_chat_template"):
            msgs = r.get("messages") or [{"role": "user", "content": r["instruction"]},
                                         {"role": "assistant", "content": r["response"]}]
            full = self.tok.apply_chat_template(msgs, tokenize=True)
            prompt = self.tok.apply_chat_template(msgs[:-1], tokenize=True, add_generation_prompt=True)
            p_ids, f_ids = list(prompt), list(full)
        else:
            p_ids = self.tok.encode(PROMPT_TEMPLATE.format(instruction=r["instruction"]), add_special_tokens=False)
            r_ids = self.tok.encode(r["response"], add_special_tokens=False)
            f_ids = list(p_ids) + list(r_ids) + ([eos] if eos is not None else [])
        if len(f_ids) > self.max_seq_len:
            if not self.truncate or len(p_ids) >= self.max_seq_len:
                return None
            f_ids = f_ids[: self.max_seq_len]
        if len(f_ids) < getattr(self, "min_seq_len", 0):
            return None
        toks = torch.tensor(f_ids, dtype=torch.int64)
        tgt = torch.roll(toks, -1)
        tgt[-1] = IGNORE
        tgt[: max(len(p_ids) - 1, 0)] = IGNORE        # positions whose next token is still prompt
        return Sequence(toks, targets=tgt)

    def _producer(self):
        sid = 0
        while not self._stop.is_set():
            for rec in self.records:
                if self._stop.is_set():
                    return
                s = self.encode(rec)
                if s is None:
                    self.dropped += 1
                    continue
                s.seq_id = sid
                sid += 1
                self._q.put(s)
            if not self.loop:
                self._q.put(None)
                return

    def _consume(self):
        while True:
            s = self._q.get()
            if s is None:
                return
            yield s

    def close(self):
        self._stop.set()


class CustomSchemaTokenSource(_QueueMixin):
    """Any record stream with a user function ``extract(record)`` that returns a :class:`Sequence`, ``None`` to skip
    the record, or, when a ``tokenizer`` is given, a ``(prompt_text, response_text)`` pair that is tokenised like an
    SFT record with the prompt masked (flextrain/io/sources.py:1017-1100).  ``records`` may be a list (``loop=True``
    cycles it, :meth:`reset` rewinds it) or any iterator (consumed lazily, once)."""

    def __init__(self, records: Iterable, extract: Callable, *, loop: bool = False, tokenizer=None,
                 max_seq_len: int = 2048):
        self.records, self.extract, self.loop = records, extract, loop
        self._sft = None
        if tokenizer is not None:
            self._sft = JsonSFTTokenSource.__new__(JsonSFTTokenSource)
            self._sft.tok, self._sft.max_seq_len, self._sft.chat, self._sft.truncate = tokenizer, max_seq_len, False, False
        self.skipped = 0
        self.reset()

    def reset(self) -> None:
        self._init_queue()
        self._it = self._generate()

    def _generate(self):
        sid = 0
        rewindable = isinstance(self.records, (list, tuple))
        while True:
            emitted = 0
            for rec in self.records:
                s = self.extract(rec)
                if s is not None and not isinstance(s, Sequence):
                    if self._sft is None:
                        raise TypeError("extract() must return a Sequence or None (or a (prompt, response) pair when "
                                        "the source was given a tokenizer)")
                    p, r = s
                    s = self._sft.encode({"instruction": p, "output": r})
                if s is None:
                    self.skipped += 1
                    continue
                s.seq_id = sid
                sid += 1
                emitted += 1
                yield s
            if not (self.loop and rewindable and emitted):
                return


class HFTokenSource(_QueueMixin):
    """HuggingFace ``datasets`` adapter (flextrain/io/sources.py:1108-1232): one sequence per document of
    ``text_field``, tokenised without special tokens, shorter than ``min_seq_len`` skipped, longer than ``max_seq_len``
    truncated.  With ``seq_len`` the documents are instead joined by the end-of-text token and cut into fixed windows
    with next-token targets (pre-training on a packed stream).  ``tokenizer`` is a tokenizer object or a model
    directory / hub id; ``dataset`` a hub id, a local dataset directory, or a builder name such as ``"json"`` with
    ``data_files``.  Needs the ``datasets`` package, and the network or a local copy of the data."""

    def __init__(self, dataset: str, tokenizer="gpt2", seq_len: Optional[int] = None, split: str = "train",
                 text_column: Optional[str] = None, name: Optional[str] = None, *, subset: Optional[str] = None,
                 text_field: str = "text", min_seq_len: int = 32, max_seq_len: int = 2048, streaming: bool = True,
                 trust_remote_code: bool = False, data_files=None):
        try:
            import datasets
        except ImportError as e:   # pragma: no cover
            raise ImportError("HFTokenSource needs the `datasets` package") from e
        kw = dict(split=split, streaming=streaming)
        if data_files is not None:
            kw["data_files"] = data_files
        if trust_remote_code:
            kw["trust_remote_code"] = True
        self.ds = datasets.load_dataset(dataset, subset or name, **kw)
        if isinstance(tokenizer, str):
            from transformers import AutoTokenizer
            tokenizer = AutoTokenizer.from_pretrained(tokenizer, trust_remote_code=trust_remote_code)
        self.tok, self.seq_len, self.col = tokenizer, seq_len, text_column or text_field
        self.min_seq_len, self.max_seq_len = int(min_seq_len), int(max_seq_len)
        self._init_queue()
        self._it = self._windows() if seq_len is not None else self._documents()

    def _ids(self, text: str) -> List[int]:
        try:
            return list(self.tok.encode(text, add_special_tokens=False))
        except TypeError:                                       # a bare tokenizer without that keyword
            return list(self.tok.encode(text))

    def _documents(self):
        sid = 0
        for row in self.ds:
            text = row.get(self.col) if hasattr(row, "get") else row[self.col]
            if not text:
                continue
            ids = self._ids(text)
            if len(ids) < self.min_seq_len:
                continue
            yield Sequence(torch.tensor(ids[: self.max_seq_len], dtype=torch.int64), seq_id=sid)
            sid += 1

    def _windows(self):
        buf: List[int] = []
        sid = 0
        for row in self.ds:
            buf += self._ids(row[self.col]) + [self.tok.eos_token_id or 0]
            while len(buf) > self.seq_len:
                win = torch.tensor(buf[: self.seq_len + 1], dtype=torch.int64)
                buf = buf[self.seq_len:]
                yield Sequence(win[:-1].clone(), targets=win[1:].clone(), seq_id=sid)
                sid += 1
