"""Synthetic packed SFT data: documents of Zipf-distributed text ids and uniform
[-1, 1] images, mixed between understanding samples (image(s) + question + answer
with loss) and text-to-image samples (prompt + generation image with flow-matching
loss), packed to a fixed token budget.  Stands in for the streaming multimodal
datasets of the reference (training/sensenovavl/data/multimodal_dataset.py:59-947)
where no dataset or tokenizer files exist."""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch

from ..config import ModelConfig
from .batch import PackedBatch, Sample, Segment, build_packed_batch

RESERVED_IDS = 8  # ids below this are special tokens (<IMG_CONTEXT>, <img>, </img>, ...)


def zipf_ids(n: int, vocab: int, a: float, gen: torch.Generator) -> torch.Tensor:
    """n ids with P(rank r) ~ r^-a over [RESERVED_IDS, vocab)."""
    u = torch.rand(n, generator=gen, dtype=torch.float64)
    m = vocab - RESERVED_IDS
    if abs(a - 1.0) < 1e-9:
        r = torch.exp(u * math.log(m))
    else:
        r = ((m ** (1 - a) - 1) * u + 1) ** (1 / (1 - a))
    return (r.floor().clamp(1, m).long() - 1) + RESERVED_IDS


def synthetic_samples(cfg: ModelConfig, token_budget: int, seed: int = 0, text_frac: float = 0.6,
                      image_sizes: Sequence[int] = (512, 768, 1024), max_images: int = 4,
                      gen_frac: float = 0.5, zipf_a: float = 1.1) -> List[Sample]:
    """Samples whose packed length (including image delimiter tokens) stays within
    ``token_budget`` and whose partitions still fit after 128-row padding."""
    gen = torch.Generator().manual_seed(seed)
    tp = cfg.token_pixels
    samples: List[Sample] = []
    used_gen = used_und = 0

    def fits(g, u):
        pad = lambda n: (n + 127) // 128 * 128
        return pad(used_gen + g) + pad(used_und + u) <= token_budget

    guard = 0
    while guard < 10000:
        guard += 1
        n_img = int(torch.randint(1, max_images + 1, (1,), generator=gen))
        is_gen = bool(torch.rand(1, generator=gen) < gen_frac)
        sizes = [int(image_sizes[int(torch.randint(0, len(image_sizes), (1,), generator=gen))])
                 for _ in range(n_img)]
        if is_gen:
            sizes = sizes[:1]
        img_tokens = sum((s // tp) ** 2 for s in sizes)
        n_text = max(16, int(img_tokens * text_frac / max(1e-6, 1 - text_frac)))
        g_add = img_tokens if is_gen else 0
        u_add = n_text + 2 * len(sizes) + (0 if is_gen else img_tokens)
        if not fits(g_add, u_add):
            # shrink to a text-only tail that fills what is left, then stop
            pad = lambda n: (n + 127) // 128 * 128
            left = token_budget - pad(used_gen) - used_und
            if left >= 8:
                ids = zipf_ids(left, cfg.vocab_size, zipf_a, gen)
                samples.append(Sample([Segment("text", ids=ids, loss=True)]))
                used_und += left
            break
        segs: List[Segment] = []
        if is_gen:
            segs.append(Segment("text", ids=zipf_ids(n_text, cfg.vocab_size, zipf_a, gen), loss=False))
            px = torch.rand(3, sizes[0], sizes[0], generator=gen) * 2 - 1
            segs.append(Segment("gen_image", pixels=px))
            samples.append(Sample(segs, task=3))
        else:
            q = n_text // 3
            for s in sizes:
                segs.append(Segment("und_image", pixels=torch.rand(3, s, s, generator=gen) * 2 - 1))
            segs.append(Segment("text", ids=zipf_ids(q, cfg.vocab_size, zipf_a, gen), loss=False))
            segs.append(Segment("text", ids=zipf_ids(n_text - q, cfg.vocab_size, zipf_a, gen), loss=True))
            samples.append(Sample(segs, task=0))
        used_gen += g_add
        used_und += u_add
    return samples


def synthetic_batch(cfg: ModelConfig, seq_len: int, seed: int = 0, **kw) -> PackedBatch:
    samples = synthetic_samples(cfg, seq_len, seed=seed, **kw)
    return build_packed_batch(samples, cfg, seq_len=seq_len, seed=seed)


def interleaved_batch(cfg: ModelConfig, seq_len: int, seed: int = 0, num_images: int = 8, image_px: int = 512,
                      zipf_a: float = 1.1) -> PackedBatch:
    """One long interleaved document: ``num_images`` images of ``image_px`` x ``image_px`` (understanding and
    generation images alternating) between Zipf text segments, filling ``seq_len`` tokens (the long-context
    configuration: 32768 tokens, 8 images of 512 x 512)."""
    gen = torch.Generator().manual_seed(seed)
    tp = cfg.token_pixels
    T = (image_px // tp) ** 2
    n_gen = num_images // 2
    pad = lambda n: (n + 127) // 128 * 128
    text_total = seq_len - pad(n_gen * T) - (num_images - n_gen) * T - 2 * num_images - 128
    per = max(16, text_total // (num_images + 1))
    segs: List[Segment] = []
    for i in range(num_images):
        segs.append(Segment("text", ids=zipf_ids(per, cfg.vocab_size, zipf_a, gen), loss=i > 0))
        px = torch.rand(3, image_px, image_px, generator=gen) * 2 - 1
        segs.append(Segment("gen_image" if i % 2 else "und_image", pixels=px))
    segs.append(Segment("text", ids=zipf_ids(per, cfg.vocab_size, zipf_a, gen), loss=True))
    return build_packed_batch([Sample(segs, task=5)], cfg, seq_len=seq_len, seed=seed)


def tiny_batch(cfg: ModelConfig, seed: int = 0, n_text: int = 128, image_px: Optional[int] = None,
               seq_len: Optional[int] = None, with_und_image: bool = False) -> PackedBatch:
    """One packed sequence: ``n_text`` uniform text ids and one generation image
    (default 8x8 = 64 tokens); optionally one understanding image as well."""
    gen = torch.Generator().manual_seed(seed)
    px = image_px or 8 * cfg.token_pixels
    ids = torch.randint(RESERVED_IDS, cfg.vocab_size, (n_text,), generator=gen)
    segs = []
    if with_und_image:
        segs.append(Segment("und_image", pixels=torch.rand(3, px, px, generator=gen) * 2 - 1))
    segs += [Segment("text", ids=ids[: n_text // 2], loss=False),
             Segment("text", ids=ids[n_text // 2:], loss=True),
             Segment("gen_image", pixels=torch.rand(3, px, px, generator=gen) * 2 - 1)]
    return build_packed_batch([Sample(segs, task=3)], cfg, seq_len=seq_len, seed=seed)
