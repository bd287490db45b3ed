#!/usr/bin/env python
"""Image editing CLI (flags of the reference example, examples/editing/inference.py:204-520).

    python examples/editing/inference.py --model_path CKPT --image in.png --prompt "make the sky purple"
    python examples/editing/inference.py --model_path CKPT --jsonl edits.jsonl --output_dir outputs --compare
    python examples/editing/inference.py --random_init tiny-mot --prompt "anything" --image_size 256    # no checkpoint
"""
import argparse
import math
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

DEFAULT_TARGET_PIXELS = 2048 * 2048


def input_pixel_budget(spec, n_images: int) -> int:
    """``auto``: up to two inputs at 2048 x 2048, that total divided across more; otherwise the integer given."""
    if str(spec) == "auto":
        return DEFAULT_TARGET_PIXELS if n_images <= 2 else 2 * DEFAULT_TARGET_PIXELS // n_images
    return int(spec)


def output_size(first_hw, target_pixels: int, factor: int):
    """Keeps the first input's aspect ratio and rescales H*W to ``target_pixels`` (sides multiples of ``factor``)."""
    h, w = first_hw
    s = math.sqrt(target_pixels / float(h * w))
    snap = lambda v: max(factor, int(round(v * s / factor)) * factor)
    return snap(w), snap(h)


def compare_sheet(inputs, edited):
    """PIL sheet: the input images (ImageNet-normalised tensors) and the edited one ([-1, 1]) side by side."""
    import torch
    from sensenova_u1_b200.utils.comparison import comparison_sheet
    mean = torch.tensor([0.485, 0.456, 0.406]).view(3, 1, 1)
    std = torch.tensor([0.229, 0.224, 0.225]).view(3, 1, 1)
    ins = [((im.float().cpu() * std + mean) * 2 - 1).clamp(-1, 1) for im in inputs]
    return comparison_sheet(ins + [edited.float().cpu()], [f"input {i}" for i in range(len(ins))] + ["edited"])


def parse(argv=None):
    from sensenova_u1_b200.utils import cli
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    cli.add_model_args(ap)
    ap.add_argument("--prompt", default=None, help="edit instruction")
    ap.add_argument("--jsonl", default=None, help='one edit per line: {"prompt": ..., "image": path or [paths]}, optionally '
                                                  '"width", "height", "seed", "output"')
    ap.add_argument("--image", nargs="+", action="extend", default=[], help="input image path(s)")
    ap.add_argument("--image_size", type=int, default=512, help="side of the synthetic input when no --image is given")
    ap.add_argument("--output", default="output.png")
    ap.add_argument("--output_dir", default="outputs")
    ap.add_argument("--width", type=int, default=None)
    ap.add_argument("--height", type=int, default=None)
    ap.add_argument("--target_pixels", type=int, default=DEFAULT_TARGET_PIXELS,
                    help="pixel count of the output when --width / --height are not given (first input's aspect ratio)")
    ap.add_argument("--input_max_pixels", "--max_input_pixels", dest="input_max_pixels", default="auto",
                    help="pixel budget per input image (integer) or auto")
    ap.add_argument("--do_resize", "--do-resize", dest="do_resize", action=argparse.BooleanOptionalAction, default=True,
                    help="resize the inputs to the input pixel budget before the model's own preprocessing")
    cli.add_sampling_args(ap)
    ap.add_argument("--img_cfg_scale", type=float, default=1.0)
    ap.add_argument("--think", action="store_true", help="accepted for compatibility: editing prompts carry an empty think block")
    ap.add_argument("--use_edit_pe", "--use-edit-pe", dest="use_edit_pe", action="store_true",
                    help="rewrite the instruction with the edit-instruction enhancer first")
    ap.add_argument("--print_edit_pe", "--print-edit-pe", dest="print_edit_pe", action="store_true")
    ap.add_argument("--edit_pe_model", "--edit-pe-model", dest="edit_pe_model", default=None,
                    help="model name for the enhancer (default: U1_ENHANCE_MODEL)")
    ap.add_argument("--compare", action="store_true", help="also write <output>_compare.png: inputs and result side by side")
    a = ap.parse_args(argv)
    if not (a.prompt or a.jsonl):
        a.prompt = "make the sky purple"
    if a.prompt and a.jsonl:
        ap.error("--prompt and --jsonl exclude each other")
    return a


def main(argv=None):
    a = parse(argv)
    import torch
    from sensenova_u1_b200.inference.images import load_image_native
    from sensenova_u1_b200.utils import cli
    from sensenova_u1_b200.utils.profiler import InferenceProfiler
    prof = InferenceProfiler(enabled=a.profile)
    with prof.time_load():
        model, tok = cli.load_from_args(a)
    f = model.cfg.token_pixels
    rewriter = None
    if a.use_edit_pe:
        from sensenova_u1_b200.inference.prompt_enhance import backend_from_env
        from sensenova_u1_b200.u1_5.briefs import enhance_edit_prompt
        backend = backend_from_env(model=a.edit_pe_model)
        rewriter = lambda text, imgs: enhance_edit_prompt(backend, imgs, text)
    for job, out in cli.iter_jobs(a, dict(prompt=a.prompt, image=list(a.image), width=a.width, height=a.height, seed=a.seed)):
        paths = job.get("image") or []
        paths = [paths] if isinstance(paths, str) else list(paths)
        if paths:
            from PIL import Image
            budget = input_pixel_budget(a.input_max_pixels, len(paths)) if a.do_resize else 4096 * 4096
            images = [load_image_native(Image.open(p).convert("RGB"), factor=f, max_pixels=budget) for p in paths]
        else:
            g = torch.Generator().manual_seed(int(job["seed"]))
            side = a.image_size // f * f
            images = [torch.randn(3, side, side, generator=g)]
        if job.get("width") and job.get("height"):
            size = (int(job["width"]) // f * f, int(job["height"]) // f * f)
        elif paths:
            size = output_size(images[0].shape[1:], a.target_pixels, f)
        else:
            size = (images[0].shape[2], images[0].shape[1])
        prompt = job["prompt"]
        if rewriter is not None:
            prompt = rewriter(prompt, paths)
            if a.print_edit_pe:
                print("rewritten instruction:", prompt)
        with prof.time_generate(image_tokens=(size[0] // f) * (size[1] // f) * a.batch_size):
            img = model.it2i_generate(tok, prompt, images, cfg_scale=a.cfg_scale, img_cfg_scale=a.img_cfg_scale,
                                      timestep_shift=a.timestep_shift, cfg_norm=a.cfg_norm, image_size=size,
                                      cfg_interval=tuple(a.cfg_interval), num_steps=a.num_steps,
                                      batch_size=a.batch_size, seed=int(job["seed"]))
        cli.save_images(img, out)
        if a.compare:
            compare_sheet(images, img[0]).save(out.with_name(out.stem + "_compare.png"))
    if a.profile:
        print(prof.report())
    return 0


if __name__ == "__main__":
    sys.exit(main())
