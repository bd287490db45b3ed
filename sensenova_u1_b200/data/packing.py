"""Sample packing and the streaming training loader.

``PackedDataset`` follows the behaviour of the reference's packer
(training/sensenovavl/data/dataset_interleaved_iterable.py:823-1623): samples stream in, each
goes to the open buffer that it fills best (best fit by remaining tokens, with an image-count
budget per sequence), a sample longer than what is left may be split at a text boundary, buffers
that have waited too long are flushed, and the whole thing is resumable (``state_dict``).
``RestartableLoader`` restarts a dead worker with back-off (trainer_builder.py:488-526,
build_dataloader.py:379-400); per-sample exceptions skip the sample (:945-1011).
"""
from __future__ import annotations

import json
import random
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Callable, Dict, Iterable, Iterator, List, Optional

import torch

from ..config import ModelConfig
from .batch import PackedBatch, Sample, Segment, build_packed_batch


def sample_tokens(s: Sample, cfg: ModelConfig) -> Dict[str, int]:
    """Token footprint of a sample: generation rows, understanding rows and image count."""
    g = u = imgs = 0
    tp = cfg.token_pixels
    for seg in s.segments:
        if seg.kind == "text":
            u += int(seg.ids.numel())
        else:
            t = (seg.pixels.shape[1] // tp) * (seg.pixels.shape[2] // tp)
            imgs += 1
            u += 2
            if seg.kind == "gen_image":
                g += t
                if seg.duplicate_for_und:
                    u += t + 2
                    imgs += 1
            else:
                u += t
    return {"gen": g, "und": u, "images": imgs}


def _pad128(n):
    return (n + 127) // 128 * 128


@dataclass
class _Buffer:
    samples: List[Sample] = field(default_factory=list)
    gen: int = 0
    und: int = 0
    images: int = 0
    age: int = 0

    def size_with(self, t) -> int:
        return _pad128(self.gen + t["gen"]) + _pad128(self.und + t["und"])


def split_text_tail(s: Sample, budget_und: int):
    """Splits a sample at a text boundary so that the head has at most ``budget_und`` understanding
    tokens; images are never cut.  Returns (head or None, tail or None)."""
    head, tail, used = [], [], 0
    for i, seg in enumerate(s.segments):
        n = int(seg.ids.numel()) if seg.kind == "text" else None
        if tail:
            tail.append(seg)
            continue
        if seg.kind != "text":
            tail = list(s.segments[i:])
            break
        if used + n <= budget_und:
            head.append(seg); used += n
        else:
            keep = budget_und - used
            if keep > 0:
                head.append(Segment("text", ids=seg.ids[:keep], loss=seg.loss))
                tail.append(Segment("text", ids=seg.ids[keep:], loss=seg.loss))
            else:
                tail.append(seg)
            tail += list(s.segments[i + 1:])
            break
    return (Sample(head, s.task) if head else None), (Sample(tail, s.task) if tail else None)


class PackedDataset:
    def __init__(self, source: Iterable[Sample], cfg: ModelConfig, max_packed_tokens: int,
                 num_images_expected: int = 144, max_buffer_size: int = 10, max_age: int = 64,
                 allow_split: bool = True, seed: int = 0, loss_reduction: str = "square"):
        self.source, self.cfg = source, cfg
        self.loss_reduction = loss_reduction       # per-token loss weight of a sample: token / sample / square (data.loss_reduction)
        self.cap, self.max_images = max_packed_tokens, num_images_expected
        self.max_buffers, self.max_age, self.allow_split = max_buffer_size, max_age, allow_split
        self.buffers: List[_Buffer] = []
        self.consumed = 0
        self.emitted = 0
        self.seed = seed

    def _fits(self, b: _Buffer, t) -> bool:
        return b.size_with(t) <= self.cap and b.images + t["images"] <= self.max_images

    def _place(self, s: Sample) -> Optional[_Buffer]:
        t = sample_tokens(s, self.cfg)
        if _pad128(t["gen"]) + _pad128(t["und"]) > self.cap or t["images"] > self.max_images:
            return None  # can never fit: the caller drops (or splits) it
        best, best_left = None, None
        for b in self.buffers:
            if self._fits(b, t):
                left = self.cap - b.size_with(t)
                if best is None or left < best_left:
                    best, best_left = b, left
        if best is None:
            best = _Buffer()
            self.buffers.append(best)
        best.samples.append(s)
        best.gen += t["gen"]; best.und += t["und"]; best.images += t["images"]
        return best

    def _pop_ready(self, force: bool = False) -> Optional[_Buffer]:
        if not self.buffers:
            return None
        for b in self.buffers:
            b.age += 1
        full = [b for b in self.buffers if self.cap - (_pad128(b.gen) + _pad128(b.und)) < 128]
        old = [b for b in self.buffers if b.age > self.max_age]
        pick = (full or old or ([max(self.buffers, key=lambda b: b.gen + b.und)]
                                if (force or len(self.buffers) > self.max_buffers) else []))
        if not pick:
            return None
        b = pick[0]
        self.buffers.remove(b)
        return b

    def __iter__(self) -> Iterator[PackedBatch]:
        for s in self.source:
            self.consumed += 1
            try:
                placed = self._place(s)
                if placed is None and self.allow_split:
                    head, tail = split_text_tail(s, self.cap - 256)
                    for part in (head, tail):
                        if part is not None and part.segments:
                            self._place(part)
            except Exception:            # a broken sample must not stop the stream
                continue
            while True:
                b = self._pop_ready()
                if b is None:
                    break
                yield self._emit(b)
        while self.buffers:
            yield self._emit(self._pop_ready(force=True))

    def _emit(self, b: _Buffer) -> PackedBatch:
        self.emitted += 1
        return build_packed_batch(b.samples, self.cfg, seq_len=self.cap, seed=self.seed + self.emitted,
                                  loss_reduction=self.loss_reduction)

    def state_dict(self):
        return {"consumed": self.consumed, "emitted": self.emitted,
                "buffers": [[s for s in b.samples] for b in self.buffers]}

    def load_state_dict(self, sd):
        self.consumed, self.emitted = sd["consumed"], sd["emitted"]
        self.buffers = []
        for samples in sd["buffers"]:
            for s in samples:
                self._place(s)


class JsonlConversationSource:
    """Reads the reference's meta JSON + per-dataset jsonl annotations
    (training/README.md:193-229; multimodal_dataset.py:62-206): each line
    ``{"conversations": [{"from", "value"}], "image"|"images": [...]}`` with ``<image>`` placeholders.
    Needs a tokenizer callable ``str -> list[int]`` and an image loader ``path -> float tensor [3,H,W]`` in [-1,1]."""

    def __init__(self, meta_path: str, tokenize: Callable[[str], List[int]], load_image: Callable[[str], torch.Tensor],
                 repeat: bool = True, seed: int = 0, start: int = 0):
        self.meta = json.loads(Path(meta_path).read_text())
        self.tokenize, self.load_image = tokenize, load_image
        self.repeat, self.rng, self.pos = repeat, random.Random(seed), start

    def _records(self):
        for name, ds in self.meta.items():
            root = Path(ds.get("root", "."))
            task = {"mm_t2i": 3, "mm_it2i": 4, "mm_interleave_gen": 5}.get(ds.get("data_type", ""), 0)
            with open(ds["annotation"]) as f:
                for line in f:
                    if line.strip():
                        yield root, task, json.loads(line)

    def __iter__(self) -> Iterator[Sample]:
        n = 0
        while True:
            for root, task, rec in self._records():
                n += 1
                if n <= self.pos:
                    continue
                self.pos = n
                try:
                    yield self._to_sample(root, task, rec)
                except Exception:
                    continue
            if not self.repeat:
                return

    def _to_sample(self, root: Path, task: int, rec: dict) -> Sample:
        imgs = rec.get("images") or ([rec["image"]] if rec.get("image") else [])
        imgs = list(imgs)
        segs: List[Segment] = []
        for turn in rec["conversations"]:
            is_answer = turn["from"] in ("gpt", "assistant")
            parts = turn["value"].split("<image>")
            for i, txt in enumerate(parts):
                if i > 0:
                    px = self.load_image(str(root / imgs.pop(0)))
                    kind = "gen_image" if (is_answer and task in (3, 4, 5)) else "und_image"
                    segs.append(Segment(kind, pixels=px, duplicate_for_und=(kind == "gen_image" and task == 5)))
                if txt:
                    role = "assistant" if is_answer else turn["from"]
                    ids = self.tokenize(f"<|im_start|>{role}\n{txt}<|im_end|>\n")
                    segs.append(Segment("text", ids=torch.tensor(ids, dtype=torch.long), loss=is_answer))
        return Sample(segs, task)


class RestartableLoader:
    """Iterates ``make_iter()``; when the iterator dies it is rebuilt (with back-off) up to
    ``max_restarts`` times, so a crashed data worker does not end the run."""

    def __init__(self, make_iter: Callable[[], Iterator], max_restarts: int = 3, backoff_s: float = 0.5):
        self.make_iter, self.max_restarts, self.backoff = make_iter, max_restarts, backoff_s
        self.restarts = 0

    def __iter__(self):
        it = self.make_iter()
        while True:
            try:
                yield next(it)
            except StopIteration:
                return
            except Exception:
                self.restarts += 1
                if self.restarts > self.max_restarts:
                    raise
                time.sleep(self.backoff * self.restarts)
                it = self.make_iter()
