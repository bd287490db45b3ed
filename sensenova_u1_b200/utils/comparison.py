"""Side-by-side image comparison sheets (same job as src/sensenova_u1/utils/comparison.py:1-184):
paste several results of one prompt (different settings, seeds or checkpoints) into one labelled
picture, and report simple difference numbers between image tensors."""
from __future__ import annotations

from typing import Dict, Sequence

import torch


def difference(a: torch.Tensor, b: torch.Tensor) -> Dict[str, float]:
    """Mean absolute error, max error and PSNR (dB) of two [3,H,W] tensors in [-1, 1]."""
    a, b = a.float(), b.float()
    mse = float(((a - b) ** 2).mean())
    return {"mae": float((a - b).abs().mean()), "max": float((a - b).abs().max()),
            "psnr": float("inf") if mse == 0 else 10.0 * torch.log10(torch.tensor(4.0 / mse)).item()}


def comparison_sheet(images: Sequence[torch.Tensor], labels: Sequence[str] = (), pad: int = 8, label_h: int = 20):
    """PIL image with the inputs ([3,H,W] in [-1,1], any sizes) side by side, labels underneath."""
    from PIL import Image, ImageDraw
    from ..inference.images import to_pil
    pics = [to_pil(x) for x in images]
    H = max(p.height for p in pics)
    W = sum(p.width for p in pics) + pad * (len(pics) + 1)
    sheet = Image.new("RGB", (W, H + 2 * pad + (label_h if labels else 0)), (255, 255, 255))
    draw = ImageDraw.Draw(sheet)
    x = pad
    for i, p in enumerate(pics):
        sheet.paste(p, (x, pad))
        if labels and i < len(labels):
            draw.text((x, H + pad + 2), str(labels[i]), fill=(0, 0, 0))
        x += p.width + pad
    return sheet
