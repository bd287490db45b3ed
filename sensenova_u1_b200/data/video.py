"""Video understanding samples: a clip becomes a run of understanding images (one per sampled frame) inside the
conversation, exactly like several ``<image>`` placeholders (reference: ``video_get_item``,
training/sensenovavl/data/multimodal_dataset.py:949-1128; frame sampling ``min_num_frame`` / ``max_num_frame``,
training/sensenovavl/data/dataset.py).

No video decoder ships with this package.  ``load_frames`` reads what is available without one: a directory of
frame images, an ``.npy`` / ``.pt`` array ``[T, H, W, 3]`` or ``[T, 3, H, W]``, an animated GIF / multi-frame image
through PIL; and a container file when ``decord`` or ``cv2`` is importable.
"""
from __future__ import annotations

import random
from pathlib import Path
from typing import Callable, List, Optional, Sequence

import torch

from .batch import Sample, Segment

IMAGE_SUFFIXES = (".jpg", ".jpeg", ".png", ".bmp", ".webp")


def sample_frame_indices(num_frames: int, min_num: int = 4, max_num: int = 24, rng: Optional[random.Random] = None,
                         clip: Optional[Sequence[float]] = None, fps: float = 1.0) -> List[int]:
    """Segment-wise frame sampling: the clip (or its ``clip = (start_s, end_s)`` part) is cut into ``n`` equal
    segments, ``n`` drawn in ``[min_num, max_num]`` (capped by the frames there are), one frame from the middle of
    each segment, jittered inside the segment when ``rng`` is given (training) and centred otherwise."""
    if num_frames <= 0:
        return []
    lo, hi = 0, num_frames
    if clip is not None:
        lo = max(0, min(num_frames - 1, int(clip[0] * fps)))
        hi = max(lo + 1, min(num_frames, int(clip[1] * fps) + 1))
    span = hi - lo
    n = max(1, min(span, rng.randint(min_num, max_num) if rng is not None else max_num))
    n = max(min(min_num, span), n)
    seg = span / n
    out = []
    for i in range(n):
        a, b = lo + seg * i, lo + seg * (i + 1)
        pos = rng.uniform(a, b) if rng is not None else (a + b) / 2
        out.append(min(hi - 1, max(lo, int(pos))))
    return out


def _to_chw(frames: torch.Tensor) -> torch.Tensor:
    if frames.dim() != 4:
        raise ValueError(f"a frame array needs 4 dimensions, got {tuple(frames.shape)}")
    if frames.shape[-1] == 3 and frames.shape[1] != 3:
        frames = frames.permute(0, 3, 1, 2)
    return frames


def load_frames(path: str, indices: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Frames ``[T, 3, H, W]`` as uint8 (all of them, or ``indices``)."""
    p = Path(path)
    if p.is_dir():
        files = sorted(f for f in p.iterdir() if f.suffix.lower() in IMAGE_SUFFIXES)
        if indices is not None:
            files = [files[i] for i in indices]
        from PIL import Image
        import numpy as np
        return torch.stack([torch.from_numpy(np.asarray(Image.open(f).convert("RGB"))).permute(2, 0, 1) for f in files])
    if p.suffix == ".npy":
        import numpy as np
        fr = _to_chw(torch.from_numpy(np.load(p)))
    elif p.suffix in (".pt", ".pth"):
        fr = _to_chw(torch.load(p))
    elif p.suffix.lower() in (".gif", ".webp", ".tif", ".tiff"):
        from PIL import Image, ImageSequence
        import numpy as np
        im = Image.open(p)
        fr = torch.stack([torch.from_numpy(np.asarray(f.convert("RGB"))).permute(2, 0, 1) for f in ImageSequence.Iterator(im)])
    else:
        fr = _decode_container(p, indices)
        indices = None
    if indices is not None:
        fr = fr[torch.as_tensor(list(indices), dtype=torch.long)]
    return fr.to(torch.uint8) if fr.dtype != torch.uint8 else fr


def count_frames(path: str) -> int:
    p = Path(path)
    if p.is_dir():
        return sum(1 for f in p.iterdir() if f.suffix.lower() in IMAGE_SUFFIXES)
    return int(load_frames(path).shape[0])


def _decode_container(p: Path, indices) -> torch.Tensor:
    try:
        import decord
        vr = decord.VideoReader(str(p))
        idx = list(indices) if indices is not None else list(range(len(vr)))
        return torch.from_numpy(vr.get_batch(idx).asnumpy()).permute(0, 3, 1, 2)
    except Exception:
        pass
    try:
        import cv2
        cap = cv2.VideoCapture(str(p))
        frames, want, i = [], (set(indices) if indices is not None else None), 0
        while True:
            ok, fr = cap.read()
            if not ok:
                break
            if want is None or i in want:
                frames.append(torch.from_numpy(cv2.cvtColor(fr, cv2.COLOR_BGR2RGB)).permute(2, 0, 1))
            i += 1
        cap.release()
        if frames:
            return torch.stack(frames)
    except Exception:
        pass
    raise RuntimeError(f"{p}: no decoder for this container here (decord / cv2 missing or unable); "
                       "extract the frames to a directory or an .npy array")


def video_record_to_sample(rec: dict, tokenize: Callable[[str], List[int]], prepare_frame: Callable[[torch.Tensor], torch.Tensor],
                           root: Path = Path("."), rng: Optional[random.Random] = None, min_num_frame: int = 4,
                           max_num_frame: int = 24, und_loss: bool = True) -> Sample:
    """One video QA record ``{"video": path, "conversations": [...], "clip": [s, e]?, "fps": f?}`` -> Sample: the
    ``<video>`` (or first ``<image>``) placeholder becomes ``Frame1: <image> ... FrameN: <image>`` with one
    understanding image per sampled frame.  ``prepare_frame``: uint8 ``[3,H,W]`` -> normalised float ``[3,H',W']``
    (resize to the token grid + ImageNet normalisation)."""
    path = str(root / rec["video"])
    total = count_frames(path)
    idx = sample_frame_indices(total, min_num_frame, max_num_frame, rng, rec.get("clip"), float(rec.get("fps", 1.0)))
    frames = load_frames(path, idx)
    segs: List[Segment] = []
    used = False
    for turn in rec["conversations"]:
        is_answer = turn["from"] in ("gpt", "assistant")
        role = "assistant" if is_answer else "user"
        text = turn["value"]
        for tag in ("<video>", "<image>"):
            if not used and tag in text:
                before, after = text.split(tag, 1)
                ids = tokenize(f"<|im_start|>{role}\n{before}")
                if ids:
                    segs.append(Segment("text", ids=torch.tensor(ids, dtype=torch.long), loss=False))
                for k in range(frames.shape[0]):
                    segs.append(Segment("text", ids=torch.tensor(tokenize(f"Frame{k + 1}: "), dtype=torch.long), loss=False))
                    segs.append(Segment("und_image", pixels=prepare_frame(frames[k])))
                    segs.append(Segment("text", ids=torch.tensor(tokenize("\n"), dtype=torch.long), loss=False))
                ids = tokenize(f"{after}<|im_end|>\n")
                segs.append(Segment("text", ids=torch.tensor(ids, dtype=torch.long), loss=is_answer and und_loss))
                used = True
                break
        else:
            ids = tokenize(f"<|im_start|>{role}\n{text}<|im_end|>\n")
            segs.append(Segment("text", ids=torch.tensor(ids, dtype=torch.long), loss=is_answer and und_loss))
    return Sample(segs, 0)
