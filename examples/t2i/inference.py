#!/usr/bin/env python
"""Text-to-image CLI (flags of the reference example, examples/t2i/inference.py:196-348).

    python examples/t2i/inference.py --model_path CKPT --prompt "..." --width 2048 --height 2048
    python examples/t2i/inference.py --model_path CKPT --jsonl prompts.jsonl --output_dir outputs
    python examples/t2i/inference.py --random_init 8b-mot --prompt_tokens 256 --profile   # no checkpoint needed
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 examples/t2i/inference.py ...
        # 2 ranks: one per guidance branch; 4 / 8 ranks: also 2 / 4 token slices per branch
"""
import argparse
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))


def parse(argv=None):
    from sensenova_u1_b200.utils import cli
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    cli.add_model_args(ap)
    ap.add_argument("--prompt", default=None, help="generate from one prompt")
    ap.add_argument("--jsonl", default=None,
                    help='one sample per line: {"prompt": ...} and optionally "width", "height", "seed", "output"')
    ap.add_argument("--prompt_tokens", type=int, default=0, help="use this many random token ids as the prompt")
    ap.add_argument("--output", default="output.png", help="output path with --prompt")
    ap.add_argument("--output_dir", default="outputs", help="output directory with --jsonl")
    ap.add_argument("--width", type=int, default=2048)
    ap.add_argument("--height", type=int, default=2048)
    cli.add_sampling_args(ap)
    ap.add_argument("--enhance", action="store_true",
                    help="rewrite the prompt with an LLM first (U1_ENHANCE_{BACKEND,ENDPOINT,API_KEY,MODEL})")
    ap.add_argument("--print_enhance", action="store_true")
    ap.add_argument("--think", action="store_true", help="the model writes a <think> block before drawing")
    ap.add_argument("--think_output", default=None, help="where the reasoning text goes (default: <output>.think.txt)")
    ap.add_argument("--print_think", action="store_true")
    a = ap.parse_args(argv)
    if not (a.prompt or a.jsonl or a.prompt_tokens):
        a.prompt = "a photo of a cat"
    if a.prompt and a.jsonl:
        ap.error("--prompt and --jsonl exclude each other")
    return a


def main(argv=None):
    a = parse(argv)
    import torch
    from sensenova_u1_b200.inference.parallel import apply_to_model, init_sampling_groups
    from sensenova_u1_b200.utils import cli
    from sensenova_u1_b200.utils.profiler import InferenceProfiler
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    groups = init_sampling_groups(2, torch.device("cuda", local))
    if "WORLD_SIZE" in os.environ and int(os.environ["WORLD_SIZE"]) > 1:
        a.device = f"cuda:{local}"
    prof = InferenceProfiler(enabled=a.profile and groups.rank == 0)
    with prof.time_load():
        model, tok = cli.load_from_args(a)
    impl = getattr(model, "impl", model)
    apply_to_model(impl, groups)
    enhancer = cli.build_enhancer(a.enhance)
    tp = model.cfg.token_pixels
    for job, out in cli.iter_jobs(a, dict(prompt=a.prompt, width=a.width, height=a.height, seed=a.seed)):
        w, h, seed = int(job["width"]), int(job["height"]), int(job["seed"])
        cli.warn_if_unsupported_resolution(w, h)
        with prof.time_generate(image_tokens=(w // tp) * (h // tp) * a.batch_size):
            if a.prompt_tokens:
                g = torch.Generator().manual_seed(seed)
                cond = torch.randint(8, model.cfg.vocab_size, (a.prompt_tokens,), generator=g)
                uncond = torch.randint(8, model.cfg.vocab_size, (8,), generator=g)
                img = impl.engine.t2i(cond, uncond, image_size=(w, h), num_steps=a.num_steps, cfg_scale=a.cfg_scale,
                                      timestep_shift=a.timestep_shift, cfg_norm=a.cfg_norm, seed=seed,
                                      cfg_interval=tuple(a.cfg_interval), batch_size=a.batch_size,
                                      cfg_group=impl.cfg_group, par_group=impl.par_group)
                thought = ""
            else:
                prompt = cli.maybe_enhance(enhancer, job["prompt"], verbose=a.print_enhance)
                res = model.t2i_generate(tok, prompt, cfg_scale=a.cfg_scale, timestep_shift=a.timestep_shift,
                                         cfg_norm=a.cfg_norm, cfg_interval=tuple(a.cfg_interval), image_size=(w, h),
                                         num_steps=a.num_steps, batch_size=a.batch_size, seed=seed, think_mode=a.think)
                img, thought = res if a.think else (res, "")
        if groups.rank != 0:                  # every rank holds the same image
            continue
        cli.save_images(img, out)
        if a.think:
            tpath = Path(a.think_output) if (a.think_output and not a.jsonl) else out.with_suffix(".think.txt")
            tpath.write_text(thought, encoding="utf-8")
            if a.print_think:
                print("think:", thought)
    if a.profile and groups.rank == 0:
        print(prof.report())
    return 0


if __name__ == "__main__":
    sys.exit(main())
