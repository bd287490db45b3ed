#!/usr/bin/env python
"""Text-to-image CLI (flags follow the reference example, examples/t2i/inference.py:196-348).

    python examples/t2i/inference.py --model_path CKPT --prompt "..." --width 2048 --height 2048
    python examples/t2i/inference.py --random_init 8b-mot --prompt_tokens 256 --profile   # no checkpoint needed
    python -m torch.distributed.run --nproc-per-node 4 --master-addr 127.0.0.1 examples/t2i/inference.py ...
        # 2 ranks: one per guidance branch; 4 / 8 ranks: also 2 / 4 token slices per branch
"""
import argparse
import os
import sys
import time

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_path", default=None)
    ap.add_argument("--random_init", default=None, help="model preset for a random-weight run (e.g. 8b-mot)")
    ap.add_argument("--prompt", default="a photo of a cat")
    ap.add_argument("--prompt_tokens", type=int, default=0, help="use this many random token ids as the prompt")
    ap.add_argument("--width", type=int, default=2048)
    ap.add_argument("--height", type=int, default=2048)
    ap.add_argument("--num_steps", type=int, default=50)
    ap.add_argument("--cfg_scale", type=float, default=4.0)
    ap.add_argument("--cfg_norm", default="none", choices=["none", "global", "channel", "cfg_zero_star"])
    ap.add_argument("--timestep_shift", type=float, default=3.0)
    ap.add_argument("--batch_size", type=int, default=1)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--think", action="store_true")
    ap.add_argument("--output", default="output.png")
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--vram_mode", default="full", choices=["full", "fast", "balanced", "low"],
                    help="full: all weights resident; others stream decoder layers from pinned host memory")
    ap.add_argument("--layers", type=int, default=None)
    a = ap.parse_args(argv)
    import torch
    from sensenova_u1_b200.config import get_config
    from sensenova_u1_b200.inference.api import ByteTokenizer, NEOChatModel
    from sensenova_u1_b200.inference.images import to_pil
    from sensenova_u1_b200.utils.profiler import InferenceProfiler
    from sensenova_u1_b200.inference.parallel import apply_to_model, init_sampling_groups
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    groups = init_sampling_groups(2, torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))))
    prof = InferenceProfiler(enabled=a.profile and groups.rank == 0)
    with prof.time_load():
        if a.model_path:
            from transformers import AutoTokenizer
            model = NEOChatModel.from_pretrained(a.model_path, vram_mode=a.vram_mode)
            tok = AutoTokenizer.from_pretrained(a.model_path, trust_remote_code=True)
        else:
            kw = {"num_layers": a.layers} if a.layers else {}
            model = NEOChatModel.from_config(get_config(a.random_init or "8b-mot", **kw), vram_mode=a.vram_mode)
            tok = ByteTokenizer(model.cfg.vocab_size)
    apply_to_model(model, groups)
    tokens = (a.width // model.cfg.token_pixels) * (a.height // model.cfg.token_pixels) * a.batch_size
    with prof.time_generate(image_tokens=tokens):
        if a.prompt_tokens:
            g = torch.Generator().manual_seed(a.seed)
            cond = torch.randint(8, model.cfg.vocab_size, (a.prompt_tokens,), generator=g)
            uncond = torch.randint(8, model.cfg.vocab_size, (8,), generator=g)
            img = model.engine.t2i(cond, uncond, image_size=(a.width, a.height), num_steps=a.num_steps,
                                   cfg_scale=a.cfg_scale, timestep_shift=a.timestep_shift, cfg_norm=a.cfg_norm,
                                   seed=a.seed, batch_size=a.batch_size, cfg_group=model.cfg_group,
                                   par_group=model.par_group)
        else:
            img = model.t2i_generate(tok, a.prompt, cfg_scale=a.cfg_scale, timestep_shift=a.timestep_shift,
                                     cfg_norm=a.cfg_norm, image_size=(a.width, a.height), num_steps=a.num_steps,
                                     batch_size=a.batch_size, seed=a.seed, think_mode=a.think)
            if a.think:
                img, thought = img
                print("think:", thought)
    if groups.rank != 0:                  # every rank holds the same image
        return 0
    for i in range(img.shape[0]):
        name = a.output if img.shape[0] == 1 else a.output.replace(".png", f"_{i}.png")
        to_pil(img[i]).save(name)
    if a.profile:
        print(prof.report())
    return 0


if __name__ == "__main__":
    sys.exit(main())
