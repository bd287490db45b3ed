#!/usr/bin/env python
"""Generation side of the image benchmarks: read a prompt list, sample N images per prompt with fixed
settings, and write the images plus one metadata record per prompt in the layout the benchmark
judges consume (``<out>/<index>/samples/<k>.png`` + ``metadata.rank<r>.jsonl``; GenEval / DPG style).  The
reference drives its benchmarks the same way (evaluation/gen/*/gen_images_*.py) and scores them with VLM
judges over HTTP; the scoring side here is ``evaluation/gen/judge_images.py``.

    python evaluation/generate_for_benchmark.py --model_path CKPT --prompts prompts.jsonl --out runs/geneval
    python evaluation/generate_for_benchmark.py --random_init tiny-mot --prompts prompts.txt --out /tmp/e --num_steps 4

``prompts``: a ``.txt`` file (one prompt per line) or ``.jsonl`` with a ``prompt`` field (other fields are
copied into the metadata).  Ranks of a torchrun launch split the prompt list (rank r takes every
world-th prompt), so an 8-GPU node generates 8 prompts at a time.
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))


def read_prompts(path):
    out = []
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            if path.endswith(".jsonl"):
                rec = json.loads(line)
                out.append(rec if "prompt" in rec else {"prompt": rec.get("text", "")})
            else:
                out.append({"prompt": line})
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model_path", default=None)
    ap.add_argument("--random_init", default=None)
    ap.add_argument("--prompts", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--n", type=int, default=4, help="images per prompt")
    ap.add_argument("--width", type=int, default=1024)
    ap.add_argument("--height", type=int, default=1024)
    ap.add_argument("--num_steps", type=int, default=50)
    ap.add_argument("--cfg_scale", type=float, default=4.0)
    ap.add_argument("--timestep_shift", type=float, default=3.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--layers", type=int, default=None)
    a = ap.parse_args(argv)
    import torch
    from sensenova_u1_b200.config import get_config
    from sensenova_u1_b200.inference.api import ByteTokenizer, NEOChatModel
    from sensenova_u1_b200.inference.images import to_pil
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if torch.cuda.is_available():
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    if a.model_path:
        from transformers import AutoTokenizer
        model = NEOChatModel.from_pretrained(a.model_path)
        tok = AutoTokenizer.from_pretrained(a.model_path, trust_remote_code=True)
    else:
        kw = {"num_layers": a.layers} if a.layers else {}
        model = NEOChatModel.from_config(get_config(a.random_init or "8b-mot", **kw))
        tok = ByteTokenizer(model.cfg.vocab_size)
    prompts = read_prompts(a.prompts)
    os.makedirs(a.out, exist_ok=True)
    done = 0
    with open(os.path.join(a.out, f"metadata.rank{rank}.jsonl"), "w") as meta:
        for i in range(rank, len(prompts), world):
            rec = prompts[i]
            d = os.path.join(a.out, f"{i:05d}", "samples")
            os.makedirs(d, exist_ok=True)
            img = model.t2i_generate(tok, rec["prompt"], cfg_scale=a.cfg_scale, timestep_shift=a.timestep_shift,
                                     image_size=(a.width, a.height), num_steps=a.num_steps, batch_size=a.n,
                                     seed=a.seed + i)
            for k in range(img.shape[0]):
                to_pil(img[k]).save(os.path.join(d, f"{k:04d}.png"))
            meta.write(json.dumps(dict(rec, index=i, samples=a.n, seed=a.seed + i, steps=a.num_steps,
                                       cfg_scale=a.cfg_scale, size=[a.width, a.height])) + "\n")
            done += 1
    print(f"rank {rank}: {done} prompts -> {a.out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
