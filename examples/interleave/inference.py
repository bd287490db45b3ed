#!/usr/bin/env python
"""Interleaved text + image generation CLI: the model writes text and, whenever it opens an image, a
picture is sampled and fed back as context (flags follow the reference example,
examples/interleave/inference.py:131-360).

    python examples/interleave/inference.py --model_path CKPT --prompt "Draw the three steps of ..."
    python examples/interleave/inference.py --random_init tiny --max_rounds 2 --num_steps 4    # no checkpoint
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_path", default=None)
    ap.add_argument("--random_init", default=None)
    ap.add_argument("--prompt", default="Tell a short story with two pictures.")
    ap.add_argument("--image", action="append", default=[], help="context image path (repeatable)")
    ap.add_argument("--max_rounds", type=int, default=4)
    ap.add_argument("--max_new_tokens", type=int, default=256)
    ap.add_argument("--width", type=int, default=512)
    ap.add_argument("--height", type=int, default=512)
    ap.add_argument("--num_steps", type=int, default=50)
    ap.add_argument("--cfg_scale", type=float, default=4.0)
    ap.add_argument("--img_cfg_scale", type=float, default=1.0)
    ap.add_argument("--timestep_shift", type=float, default=3.0)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--output_dir", default="interleave_out")
    ap.add_argument("--image_only", action="store_true", help="return the pictures only")
    ap.add_argument("--layers", type=int, default=None)
    a = ap.parse_args(argv)
    from sensenova_u1_b200.config import get_config
    from sensenova_u1_b200.inference.api import ByteTokenizer, NEOChatModel
    from sensenova_u1_b200.inference.images import load_image_native, to_pil
    if a.model_path:
        from transformers import AutoTokenizer
        model = NEOChatModel.from_pretrained(a.model_path)
        tok = AutoTokenizer.from_pretrained(a.model_path, trust_remote_code=True)
    else:
        kw = {"num_layers": a.layers} if a.layers else {}
        model = NEOChatModel.from_config(get_config(a.random_init or "8b-mot", **kw))
        tok = ByteTokenizer(model.cfg.vocab_size)
    images = []
    if a.image:
        from PIL import Image
        images = [load_image_native(Image.open(p).convert("RGB"), factor=model.cfg.token_pixels) for p in a.image]
    kw = dict(max_rounds=a.max_rounds, max_new_tokens=a.max_new_tokens, image_size=(a.width, a.height),
              cfg_scale=a.cfg_scale, img_cfg_scale=a.img_cfg_scale, timestep_shift=a.timestep_shift,
              num_steps=a.num_steps, seed=a.seed)
    if a.image_only:
        text, pics = "", model.interleave_gen_image_only(tok, a.prompt, images, **kw)
    else:
        text, pics = model.interleave_gen(tok, a.prompt, images, **kw)
    os.makedirs(a.output_dir, exist_ok=True)
    names = []
    for i, p in enumerate(pics):
        names.append(os.path.join(a.output_dir, f"image_{i}.png"))
        to_pil(p).save(names[-1])
    with open(os.path.join(a.output_dir, "result.json"), "w") as f:
        json.dump({"prompt": a.prompt, "text": text, "images": names}, f, indent=1)
    print(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
