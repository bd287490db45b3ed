#!/usr/bin/env python
"""Image-editing CLI: text + input image(s) -> edited image, three guidance branches
(flags follow the reference example, examples/editing/inference.py:204-420).

    python examples/editing/inference.py --model_path CKPT --image in.png --prompt "make it snow"
    python examples/editing/inference.py --random_init tiny --image_size 256 --num_steps 4   # no checkpoint
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_path", default=None)
    ap.add_argument("--random_init", default=None, help="model preset for a random-weight run")
    ap.add_argument("--image", action="append", default=[], help="input image path (repeatable)")
    ap.add_argument("--image_size", type=int, default=512, help="side of the synthetic input when no --image is given")
    ap.add_argument("--prompt", default="make the sky purple")
    ap.add_argument("--num_steps", type=int, default=50)
    ap.add_argument("--cfg_scale", type=float, default=4.0)
    ap.add_argument("--img_cfg_scale", type=float, default=1.0)
    ap.add_argument("--cfg_norm", default="none", choices=["none", "global", "channel", "cfg_zero_star"])
    ap.add_argument("--timestep_shift", type=float, default=3.0)
    ap.add_argument("--max_input_pixels", type=int, default=2048 * 2048, help="input-pixel budget per image")
    ap.add_argument("--width", type=int, default=None)
    ap.add_argument("--height", type=int, default=None)
    ap.add_argument("--batch_size", type=int, default=1)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--output", default="edited.png")
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--vram_mode", default="full", choices=["full", "fast", "balanced", "low"],
                    help="full: all weights resident; others stream decoder layers from pinned host memory")
    ap.add_argument("--layers", type=int, default=None)
    a = ap.parse_args(argv)
    import torch
    from sensenova_u1_b200.config import get_config
    from sensenova_u1_b200.inference.api import ByteTokenizer, NEOChatModel
    from sensenova_u1_b200.inference.images import load_image_native, to_pil
    from sensenova_u1_b200.utils.profiler import InferenceProfiler
    prof = InferenceProfiler(enabled=a.profile)
    with prof.time_load():
        if a.model_path:
            from transformers import AutoTokenizer
            model = NEOChatModel.from_pretrained(a.model_path, vram_mode=a.vram_mode)
            tok = AutoTokenizer.from_pretrained(a.model_path, trust_remote_code=True)
        else:
            kw = {"num_layers": a.layers} if a.layers else {}
            model = NEOChatModel.from_config(get_config(a.random_init or "8b-mot", **kw), vram_mode=a.vram_mode)
            tok = ByteTokenizer(model.cfg.vocab_size)
    f = model.cfg.token_pixels
    if a.image:
        from PIL import Image
        images = [load_image_native(Image.open(p).convert("RGB"), factor=f, max_pixels=a.max_input_pixels)
                  for p in a.image]
    else:
        g = torch.Generator().manual_seed(a.seed)
        side = a.image_size // f * f
        images = [torch.randn(3, side, side, generator=g)]
    size = (a.width or images[0].shape[2], a.height or images[0].shape[1])
    tokens = (size[0] // f) * (size[1] // f) * a.batch_size
    with prof.time_generate(image_tokens=tokens):
        img = model.it2i_generate(tok, a.prompt, images, cfg_scale=a.cfg_scale, img_cfg_scale=a.img_cfg_scale,
                                  timestep_shift=a.timestep_shift, cfg_norm=a.cfg_norm, image_size=size,
                                  num_steps=a.num_steps, batch_size=a.batch_size, seed=a.seed)
    for i in range(img.shape[0]):
        name = a.output if img.shape[0] == 1 else a.output.replace(".png", f"_{i}.png")
        to_pil(img[i]).save(name)
    if a.profile:
        print(prof.report())
    return 0


if __name__ == "__main__":
    sys.exit(main())
