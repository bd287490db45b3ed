#!/usr/bin/env python
"""Visual question answering CLI (flags of the reference example, examples/vqa/inference.py:29-288).

    python examples/vqa/inference.py --model_path CKPT --image in.png --question "what is shown?"
    python examples/vqa/inference.py --model_path CKPT --jsonl questions.jsonl --output_dir answers
    python examples/vqa/inference.py --random_init tiny-mot --question "anything"
"""
import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))


def parse(argv=None):
    from sensenova_u1_b200.utils import cli
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    cli.add_model_args(ap)
    ap.add_argument("--image", default=None, help="path of one image")
    ap.add_argument("--jsonl", default=None, help='one question per line: {"image": path, "question": ...}, optionally "id"')
    ap.add_argument("--question", default="Describe the image.")
    ap.add_argument("--output", default=None, help="file for the single answer (default: stdout)")
    ap.add_argument("--output_dir", default="outputs", help="directory for answers.jsonl with --jsonl")
    ap.add_argument("--max_pixels", type=int, default=4194304)
    ap.add_argument("--min_pixels", type=int, default=65536)
    ap.add_argument("--seed", type=int, default=42)
    cli.add_text_sampling_args(ap)
    a = ap.parse_args(argv)
    if a.image and a.jsonl:
        ap.error("--image and --jsonl exclude each other")
    if a.random_init is None and a.model_path is None:
        a.random_init = "tiny-mot"
    return a


def main(argv=None):
    a = parse(argv)
    from sensenova_u1_b200.inference.images import load_image_native
    from sensenova_u1_b200.utils import cli
    from sensenova_u1_b200.utils.profiler import InferenceProfiler
    prof = InferenceProfiler(enabled=a.profile)
    with prof.time_load():
        model, tok = cli.load_from_args(a)
    gc = cli.generation_config(a)
    f = model.cfg.token_pixels
    ask = lambda path, q: model.chat(tok, load_image_native(path, f, a.min_pixels, a.max_pixels) if path else None, q, gc)
    if a.jsonl:
        out_dir = Path(a.output_dir)
        out_dir.mkdir(parents=True, exist_ok=True)
        with open(out_dir / "answers.jsonl", "w", encoding="utf-8") as fo:
            for i, rec in enumerate(cli.read_jsonl(a.jsonl)):
                with prof.time_generate(image_tokens=0):
                    ans = ask(rec.get("image"), rec.get("question", a.question))
                fo.write(json.dumps({"id": rec.get("id", i), "question": rec.get("question", a.question), "answer": ans},
                                    ensure_ascii=False) + "\n")
                fo.flush()
    else:
        with prof.time_generate(image_tokens=0):
            ans = ask(a.image, a.question)
        if a.output:
            Path(a.output).write_text(ans, encoding="utf-8")
        else:
            print(ans)
    if a.profile:
        print(prof.report())
    return 0


if __name__ == "__main__":
    sys.exit(main())
