#!/usr/bin/env python
"""Generate and judge the image-generation benchmarks (BizGenEval, IGenBench, LongText, CVTG-2K, TIIF-Bench).

    # draw every prompt of a benchmark (ranks of a torchrun launch, or --num_shards / --shard_rank, split the list;
    # pictures that exist are skipped, so an interrupted run resumes)
    python evaluation/gen/run_benchmark.py generate bizgeneval --model_path CKPT --output_dir out/biz --data_path test.jsonl
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 evaluation/gen/run_benchmark.py generate tiif \\
        --model_path CKPT --output_dir out/tiif --input_folder data/testmini_prompts --resolution 1024

    # judge the pictures with a vision-language endpoint and write the benchmark's summary
    python evaluation/gen/run_benchmark.py evaluate bizgeneval --image_dir out/biz --output_dir out/biz_eval \\
        --data_path test.jsonl --api_base http://host/v1 --api_key KEY --judge_model MODEL --concurrency 8

One driver for the reference's per-benchmark pairs ``gen_images_*.py`` / ``eval_images_*.py`` (evaluation/gen/*); the
flag names are theirs (written with ``_`` or ``-``), the sampling defaults are those of their launcher scripts
(``run_*.sh``: CVTG draws with guidance 7 and time shift 1, TIIF with the ``global`` guidance norm)."""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path
from typing import Callable, List, Optional, Sequence

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from evaluation.common.judge import JudgeClient, ResultLog, run_parallel  # noqa: E402
from evaluation.gen.suites import SUITES, Job, Suite  # noqa: E402


def normalise_flags(argv: Sequence[str]) -> List[str]:
    """``--model-path`` and ``--model_path`` name the same flag."""
    out = []
    for s in argv:
        if s.startswith("--") and len(s) > 2:
            name, eq, val = s[2:].partition("=")
            s = "--" + name.replace("-", "_") + eq + val
        out.append(s)
    return out


def make_grid(images, rows: int, cols: int, pad: int = 2):
    """Several samples of one prompt side by side (TIIF's batch protocol)."""
    from PIL import Image
    if len(images) == 1:
        return images[0]
    if rows * cols < len(images):
        raise ValueError(f"rows * cols = {rows * cols} does not hold {len(images)} pictures")
    w, h = images[0].size
    grid = Image.new("RGB", (cols * w + (cols - 1) * pad, rows * h + (rows - 1) * pad), (0, 0, 0))
    for i, im in enumerate(images):
        r, c = divmod(i, cols)
        grid.paste(im, (c * (w + pad), r * (h + pad)))
    return grid


def shard(jobs: List[Job], rank: int, world: int, shard_rank: int = 0, num_shards: int = 1) -> List[Job]:
    if num_shards < 1 or not 0 <= shard_rank < num_shards:
        raise ValueError(f"shard_rank {shard_rank} outside [0, {num_shards})")
    return jobs[rank * num_shards + shard_rank::world * num_shards]


def generate(suite: Suite, a, draw: Optional[Callable] = None) -> dict:
    """``draw(prompt, size, a) -> list of PIL images``; default: the model named by the flags."""
    out_dir = Path(a.output_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    jobs = shard(suite.jobs(a), rank, world, a.shard_rank, a.num_shards)
    todo = [j for j in jobs if not (out_dir / j.out).exists()]
    print(f"[{suite.name}] rank {rank}/{world}: {len(jobs)} prompts, {len(jobs) - len(todo)} already drawn")
    if todo and draw is None:
        draw = model_drawer(a)
    for j in todo:
        imgs = draw(j.prompt, j.size, a)
        im = make_grid(imgs, a.rows, a.cols)
        if a.save_size and a.save_size != max(j.size):
            from PIL import Image
            s = a.save_size / max(j.size)
            im = im.resize((max(1, round(im.width * s)), max(1, round(im.height * s))), Image.Resampling.LANCZOS)
        p = out_dir / j.out
        p.parent.mkdir(parents=True, exist_ok=True)
        tmp = p.with_suffix(".tmp.png")
        im.save(tmp)
        os.replace(tmp, p)                           # a killed run leaves no half-written picture behind
        print(f"[saved] {j.key} {j.size[0]}x{j.size[1]} -> {p}")
    return {"prompts": len(jobs), "generated": len(todo), "skipped": len(jobs) - len(todo)}


def model_drawer(a) -> Callable:
    import torch
    from sensenova_u1_b200.inference.images import to_pil
    from sensenova_u1_b200.utils.cli import load_from_args, warn_if_unsupported_resolution
    if torch.cuda.is_available():
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    model, tok = load_from_args(a)
    warned = set()

    def draw(prompt, size, a):
        if size not in warned:
            warned.add(size)
            warn_if_unsupported_resolution(*size)
        img = model.t2i_generate(tok, prompt, cfg_scale=a.cfg_scale, cfg_norm=a.cfg_norm, timestep_shift=a.timestep_shift,
                                 cfg_interval=tuple(a.cfg_interval), image_size=size, num_steps=a.num_steps,
                                 batch_size=a.batch_size, seed=a.seed)
        return [to_pil(img[k]) for k in range(img.shape[0])]
    return draw


def evaluate(suite: Suite, a, client=None) -> dict:
    image_dir, out_dir = Path(a.image_dir), Path(a.output_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    client = client or JudgeClient(a.api_base, a.api_key, a.judge_model, timeout=a.timeout)
    tasks = suite.tasks(a, image_dir)
    n_prompts = len(suite.jobs(a))
    log_path = out_dir / "items.jsonl"
    if a.force_rerun and log_path.exists():
        log_path.unlink()
    log = ResultLog(log_path)
    if any("error" in r for r in log.records()):     # failed items of an earlier run are tried again
        keep = [r for r in log.records() if "error" not in r]
        log_path.write_text("".join(json.dumps(r, ensure_ascii=False) + "\n" for r in keep))
        log = ResultLog(log_path)
    print(f"[{suite.name}] {len(tasks)} pictures of {n_prompts} prompts, {sum(t['id'] in log for t in tasks)} judged before, "
          f"judge {getattr(client, 'model', '?')}, {a.concurrency} workers")
    ids = {t["id"] for t in tasks}
    records = [r for r in run_parallel(tasks, lambda t: suite.judge(client, t), log, a.concurrency) if r["id"] in ids]
    ok = [r for r in records if "error" not in r]
    for r in records:
        if "error" in r:
            print(f"[warn] {r['id']}: {r['error']}")
    if not ok:
        raise RuntimeError(f"{suite.name}: no picture could be judged")
    summary = {"benchmark": suite.name, **suite.summarize(ok, a), "judge_model": getattr(client, "model", None),
               "image_dir": str(image_dir), "judged": len(ok), "failed": len(records) - len(ok),
               "missing_images": n_prompts - len(tasks)}
    (out_dir / suite.summary_file).write_text(json.dumps(summary, ensure_ascii=False, indent=2))
    print(f"[{suite.name}] summary -> {out_dir / suite.summary_file}")
    return summary


def parser() -> argparse.ArgumentParser:
    from sensenova_u1_b200.utils.cli import add_model_args, add_sampling_args
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    for cmd in ("generate", "evaluate"):
        c = sub.add_parser(cmd)
        bs = c.add_subparsers(dest="benchmark", required=True)
        for name, suite in SUITES.items():
            p = bs.add_parser(name)
            suite.add_args(p)
            if cmd == "generate":
                p.add_argument("--output_dir", required=True)
                add_model_args(p)
                add_sampling_args(p)
                p.set_defaults(**suite.defaults)
                p.add_argument("--save_size", type=int, default=None, help="long side of the saved picture (LANCZOS)")
                p.add_argument("--rows", type=int, default=1)
                p.add_argument("--cols", type=int, default=1)
                p.add_argument("--num_shards", type=int, default=1)
                p.add_argument("--shard_rank", type=int, default=0)
            else:
                p.add_argument("--image_dir", "--sample_dir", "--result_dir", dest="image_dir", required=True)
                p.add_argument("--output_dir", required=True)
                p.add_argument("--api_base", default=None)
                p.add_argument("--api_key", default=None)
                p.add_argument("--judge_model", "--model", dest="judge_model", default=None)
                p.add_argument("--timeout", "--eval_timeout", dest="timeout", type=int, default=240)
                p.add_argument("--concurrency", type=int, default=8)
                p.add_argument("--force_rerun", action="store_true")
    return ap


def main(argv=None, draw=None, client=None):
    a = parser().parse_args(normalise_flags(sys.argv[1:] if argv is None else argv))
    suite = SUITES[a.benchmark]
    if a.cmd == "generate":
        if a.rows * a.cols < a.batch_size:
            raise SystemExit(f"--rows x --cols must hold --batch_size = {a.batch_size} pictures")
        return generate(suite, a, draw)
    return evaluate(suite, a, client)


if __name__ == "__main__":
    main()
