#!/usr/bin/env python
"""Interleaved text + image generation CLI (flags of the reference example, examples/interleave/inference.py:131-440).

    python examples/interleave/inference.py --model_path CKPT --prompt "a story in two pictures" --output_dir out
    python examples/interleave/inference.py --model_path CKPT --jsonl samples.jsonl --image_root data/
    python examples/interleave/inference.py --random_init tiny-mot --prompt "anything" --width 256 --height 256

Writes ``<stem>.txt`` (the text, pictures marked ``[image]``), ``<stem>_image_<i>.png`` and ``<stem>.json``.
"""
import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

# aspect-ratio buckets for generated pictures when no size is given (examples/interleave/inference.py:40-60)
SUPPORTED_RESOLUTIONS = {"1:1": (1024, 1024), "16:9": (1376, 768), "9:16": (768, 1376), "3:2": (1248, 832), "2:3": (832, 1248),
                         "4:3": (1184, 880), "3:4": (880, 1184), "5:4": (1136, 912), "4:5": (912, 1136), "21:9": (1536, 688),
                         "9:21": (672, 1568)}
DEFAULT_RESOLUTION = "1:1"


def parse(argv=None):
    from sensenova_u1_b200.inference import prompts
    from sensenova_u1_b200.utils import cli
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    cli.add_model_args(ap)
    ap.add_argument("--prompt", default=None)
    ap.add_argument("--jsonl", default=None, help='one sample per line: {"prompt": ...}, optionally "image": [paths], '
                                                  '"width", "height", "seed", "id"')
    ap.add_argument("--image", action="append", default=[], help="context image path (repeatable)")
    ap.add_argument("--image_root", default="", help="prefix of relative image paths in --jsonl")
    ap.add_argument("--output_dir", default="outputs")
    ap.add_argument("--stem", default="sample", help="file name stem with --prompt")
    ap.add_argument("--resolution", default=DEFAULT_RESOLUTION, choices=list(SUPPORTED_RESOLUTIONS),
                    help="aspect-ratio bucket of generated pictures; --width and --height override it")
    ap.add_argument("--width", type=int, default=None)
    ap.add_argument("--height", type=int, default=None)
    ap.add_argument("--cfg_scale", type=float, default=4.0)
    ap.add_argument("--img_cfg_scale", type=float, default=1.0)
    ap.add_argument("--cfg_norm", default="none", choices=cli.CFG_NORMS)
    ap.add_argument("--cfg_interval", type=float, nargs=2, default=[0.0, 1.0])
    ap.add_argument("--timestep_shift", type=float, default=3.0)
    ap.add_argument("--num_steps", type=int, default=50)
    ap.add_argument("--think_mode", action=argparse.BooleanOptionalAction, default=True,
                    help="let the model reason in a <think> block before answering (--no-think_mode: empty block)")
    ap.add_argument("--system_message", default=prompts.SYSTEM_MESSAGE_FOR_INTERLEAVE)
    ap.add_argument("--max_rounds", "--max_images", dest="max_rounds", type=int, default=10)
    ap.add_argument("--max_new_tokens", type=int, default=1024)
    ap.add_argument("--image_only", action="store_true", help="keep the pictures only")
    ap.add_argument("--seed", type=int, default=42)
    a = ap.parse_args(argv)
    if not (a.prompt or a.jsonl):
        a.prompt = "Tell a short story with two pictures."
    if a.prompt and a.jsonl:
        ap.error("--prompt and --jsonl exclude each other")
    return a


def main(argv=None):
    a = parse(argv)
    from sensenova_u1_b200.inference.images import load_image_native, to_pil
    from sensenova_u1_b200.utils import cli
    from sensenova_u1_b200.utils.profiler import InferenceProfiler
    prof = InferenceProfiler(enabled=a.profile)
    with prof.time_load():
        model, tok = cli.load_from_args(a)
    f = model.cfg.token_pixels
    base_w, base_h = SUPPORTED_RESOLUTIONS[a.resolution]
    out_dir = Path(a.output_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    jobs = cli.read_jsonl(a.jsonl) if a.jsonl else [dict(prompt=a.prompt, image=list(a.image), id=a.stem)]
    for i, job in enumerate(jobs):
        if "prompt" not in job:
            raise ValueError(f"{a.jsonl} line {i + 1}: missing 'prompt'")
        stem = str(job.get("id") or f"{i:05d}")
        paths = job.get("image") or []
        paths = [paths] if isinstance(paths, str) else list(paths)
        images = []
        if paths:
            from PIL import Image
            root = a.image_root if a.jsonl else ""
            images = [load_image_native(Image.open(os.path.join(root, p)).convert("RGB"), factor=f) for p in paths]
        w = int(job.get("width") or a.width or base_w) // f * f
        h = int(job.get("height") or a.height or base_h) // f * f
        kw = dict(max_rounds=a.max_rounds, max_new_tokens=a.max_new_tokens, image_size=(w, h), cfg_scale=a.cfg_scale,
                  img_cfg_scale=a.img_cfg_scale, cfg_norm=a.cfg_norm, cfg_interval=tuple(a.cfg_interval),
                  timestep_shift=a.timestep_shift, num_steps=a.num_steps, seed=int(job.get("seed", a.seed)),
                  system_message=a.system_message, think_mode=a.think_mode)
        with prof.time_generate(image_tokens=(w // f) * (h // f)):
            text, pics = model.interleave_gen(tok, job["prompt"], images, **kw)
        if a.image_only:
            text = ""
        names = []
        for k, p in enumerate(pics):
            names.append(str(out_dir / f"{stem}_image_{k}.png"))
            to_pil(p).save(names[-1])
        (out_dir / f"{stem}.txt").write_text(text, encoding="utf-8")
        (out_dir / f"{stem}.json").write_text(json.dumps({"prompt": job["prompt"], "text": text, "images": names}, indent=1,
                                                         ensure_ascii=False), encoding="utf-8")
        print(text)
    if a.profile:
        print(prof.report())
    return 0


if __name__ == "__main__":
    sys.exit(main())
