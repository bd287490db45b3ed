#!/usr/bin/env python
"""Run and score the interleaved / visual-reasoning benchmarks (RealUnify GEU and UEG, UniMMMU, BabyVision, OpenING).

    # inference: in-process model, or a served one with --base_url; ranks of a torchrun launch (or --num_shards /
    # --shard_rank) split the samples; finished samples are skipped on a re-run
    python evaluation/interleave/run_benchmark.py infer realunify --model_path CKPT --data_path GEU_step.jsonl \\
        --output_dir out/realunify --inference_mode interleave
    python evaluation/interleave/run_benchmark.py infer babyvision --base_url http://127.0.0.1:8000 \\
        --data_path meta_data.jsonl --image_root images --output_dir out/babyvision --workers 32

    # scoring: merges shard files, asks a judge where the benchmark needs one, prints the benchmark's table
    python evaluation/interleave/run_benchmark.py score realunify --run_dir out/realunify
    python evaluation/interleave/run_benchmark.py score opening --run_dir out/opening --meta_path data/OpenING \\
        --api_base http://host/v1 --api_key KEY --judge_model MODEL

One driver for the reference's ``inference_*.py`` / ``infer_*.py`` and ``calculate_score*.py`` / ``eval_*.py`` /
``merge_shards.py`` scripts (evaluation/interleave/*); flag names are theirs, written with ``_`` or ``-``."""
from __future__ import annotations

import argparse
import base64
import glob
import io
import json
import os
import sys
from pathlib import Path
from typing import Optional

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from evaluation.common.judge import JudgeClient, ResultLog, merge_shards, run_parallel  # noqa: E402
from evaluation.gen.run_benchmark import normalise_flags  # noqa: E402
from evaluation.interleave.suites import SUITES, LocalEngine, Suite  # noqa: E402


def square(v: str) -> int:
    """``1024`` or ``1024x1024``."""
    parts = str(v).lower().replace("*", "x").split("x")
    if not all(p.isdigit() and int(p) > 0 for p in parts) or len(parts) > 2 or len(set(parts)) != 1:
        raise argparse.ArgumentTypeError(f"a positive side or a square like 1024x1024, got {v!r}")
    return int(parts[0])


class ServedEngine:
    """The four engine calls over this framework's HTTP server (``/v1/images/generations``, ``/v1/images/edits``,
    ``/v1/chat/completions``)."""

    def __init__(self, base_url: str, timeout: float = 3600.0, session=None, **s):
        import requests
        self.base, self.timeout, self.s = base_url.rstrip("/"), timeout, s
        self.http = session or requests.Session()

    @staticmethod
    def _b64(im) -> str:
        buf = io.BytesIO()
        im.save(buf, format="PNG")
        return base64.b64encode(buf.getvalue()).decode()

    @staticmethod
    def _pil(b64: str):
        from PIL import Image
        return Image.open(io.BytesIO(base64.b64decode(b64.split(",", 1)[-1]))).convert("RGB")

    def _post(self, path, body):
        r = self.http.post(self.base + path, json=body, timeout=self.timeout)
        r.raise_for_status()
        return r.json()

    def _gen(self):
        return {k: self.s[k] for k in ("cfg_scale", "img_cfg_scale", "cfg_norm", "num_steps", "timestep_shift", "seed") if k in self.s}

    def t2i(self, prompt, size):
        r = self._post("/v1/images/generations", {"prompt": prompt, "size": f"{size[0]}x{size[1]}", "n": 1, **self._gen()})
        return self._pil(r["data"][0]["b64_json"])

    def edit(self, prompt, images, size):
        r = self._post("/v1/images/edits", {"prompt": prompt, "images": [self._b64(i) for i in images], "n": 1, **self._gen()})
        return self._pil(r["data"][0]["b64_json"])

    def _user(self, text, images):
        parts = [{"type": "text", "text": text}]
        parts += [{"type": "image_url", "image_url": {"url": "data:image/png;base64," + self._b64(i)}} for i in images]
        return [{"role": "user", "content": parts}]

    def ask(self, question, images=(), max_new_tokens=512, min_pixels=None, max_pixels=None, **gen):
        if min_pixels or max_pixels:
            # the picture is brought into the benchmark's pixel budget before it is sent (sides multiples of 32), as the
            # reference's clients do (BabyVision/infer_babyvision.py:355-410)
            from sensenova_u1_b200.inference.images import smart_resize
            sized = []
            for im in images:
                h, w = smart_resize(im.height, im.width, 32, min_pixels or 65536, max_pixels or 4194304)
                sized.append(im if (w, h) == im.size else im.resize((w, h)))
            images = sized
        body = {"messages": self._user(question, images), "max_tokens": max_new_tokens}
        if max_pixels:
            body.update(min_pixels=int(min_pixels or 65536), max_pixels=int(max_pixels))      # the server keeps that budget
        t = gen.get("temperature")
        if gen.get("do_sample") and t:
            body.update(temperature=float(t), top_p=float(gen.get("top_p", 1.0) or 1.0))
        if gen.get("repetition_penalty"):
            body["repetition_penalty"] = float(gen["repetition_penalty"])
        r = self._post("/v1/chat/completions", body)
        return r["choices"][0]["message"]["content"]

    def interleave(self, prompt, images, size, system=None, think=True, max_new_tokens=4096, max_images=None):
        messages = ([{"role": "system", "content": system}] if system else []) + self._user(prompt, images)
        body = {"messages": messages, "interleave": True, "max_tokens": max_new_tokens, "max_rounds": max_images or 4,
                "size": f"{size[0]}x{size[1]}", "chat_template_kwargs": {"enable_thinking": bool(think)}, **self._gen()}
        msg = self._post("/v1/chat/completions", body)["choices"][0]["message"]["content"]
        if isinstance(msg, str):
            return msg, []
        text = "\n".join(p.get("text", "") for p in msg if p.get("type") == "text")
        return text, [self._pil(p["image_url"]["url"]) for p in msg if p.get("type") == "image_url"]


def result_path(out_dir: Path, suite: Suite, shard: Optional[int]) -> Path:
    if shard is None:
        return out_dir / suite.result_file
    stem, ext = os.path.splitext(suite.result_file)
    return out_dir / "shards" / f"{stem}_shard_{shard:03d}{ext}"


def infer(suite: Suite, a, engine=None) -> dict:
    out_dir = Path(a.output_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    items = suite.load(a)
    if a.limit:
        items = items[:a.limit]
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    shard = None
    if a.num_shards is not None or a.shard_rank is not None:
        if a.num_shards is None or a.shard_rank is None or not 0 <= a.shard_rank < a.num_shards:
            raise SystemExit("--num_shards and --shard_rank go together, 0 <= shard_rank < num_shards")
        items, shard = items[a.shard_rank::a.num_shards], a.shard_rank
    elif world > 1:
        items, shard = items[rank::world], rank
    log = ResultLog(result_path(out_dir, suite, shard))
    if a.overwrite and log.path.exists():
        log.path.unlink()
        log = ResultLog(log.path)
    tasks = [{"id": str(it[suite.id_field]), "item": it} for it in items]
    todo = [t for t in tasks if t["id"] not in log]
    print(f"[{suite.name}] {len(tasks)} samples for this shard, {len(tasks) - len(todo)} done before, mode {a.inference_mode}")
    if todo and engine is None:
        engine = build_engine(a)
    before = len(log.done)

    def one(t):
        out = suite.run_one(engine, t["item"], a, out_dir)
        if "id" in out:                       # the log is keyed by "id": a dataset's own id moves aside
            out["sample_id"] = out.pop("id")
        return out
    run_parallel(tasks, one, log, a.workers)
    recs = [log.done[t["id"]] for t in tasks if t["id"] in log]
    failed = [r for r in recs if "error" in r]
    for r in failed[:20]:
        print(f"[warn] {r['id']}: {r['error']}")
    return {"samples": len(tasks), "new": len(log.done) - before, "failed": len(failed), "results": str(log.path)}


def build_engine(a):
    s = dict(cfg_scale=a.cfg_scale, img_cfg_scale=a.img_cfg_scale, cfg_norm=a.cfg_norm, cfg_interval=tuple(a.cfg_interval),
             num_steps=a.num_steps, timestep_shift=a.timestep_shift, seed=a.seed)
    if a.base_url:
        return ServedEngine(a.base_url, timeout=a.request_timeout, **s)
    import torch
    from sensenova_u1_b200.utils.cli import load_from_args
    if torch.cuda.is_available():
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    model, tok = load_from_args(a)
    return LocalEngine(model, tok, **s)


def score(suite: Suite, a, client=None) -> dict:
    run = Path(a.run_dir)
    shards = sorted(glob.glob(str(run / "shards" / "*_shard_*.jsonl")))
    if shards:
        whole = run / suite.result_file
        n = merge_shards(([whole] if whole.exists() else []) + shards, whole)
        print(f"[{suite.name}] merged {len(shards)} shard files: {n} samples")
    recs = [r for r in ResultLog(run / suite.result_file).records() if "error" not in r]
    if not recs:
        raise RuntimeError(f"no results in {run / suite.result_file}")
    if suite.needs_judge:
        client = client or JudgeClient(a.api_base, a.api_key, a.judge_model, timeout=a.timeout)
        stem = os.path.splitext(suite.result_file)[0]
        log = ResultLog(run / f"{stem}_scored.jsonl")
        if a.force_rerun and log.path.exists():
            log.path.unlink()
            log = ResultLog(log.path)
        ids = {r["id"] for r in recs}
        judged = [r for r in run_parallel(recs, lambda r: suite.judge(client, r, a), log, a.workers) if r["id"] in ids]
        bad = [r for r in judged if "error" in r]
        for r in bad[:20]:
            print(f"[warn] {r['id']}: {r['error']}")
        recs = [r for r in judged if "error" not in r]
    summary = {"benchmark": suite.name, **suite.summarize(recs, a), "samples": len(recs)}
    (run / f"{suite.name}_summary.json").write_text(json.dumps(summary, ensure_ascii=False, indent=2))
    print(json.dumps({k: v for k, v in summary.items() if not isinstance(v, (list,))}, ensure_ascii=False, indent=1)[:4000])
    return summary


def parser() -> argparse.ArgumentParser:
    from sensenova_u1_b200.utils.cli import add_model_args, add_sampling_args
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    sub = ap.add_subparsers(dest="cmd", required=True)
    for cmd in ("infer", "score"):
        bs = sub.add_parser(cmd).add_subparsers(dest="benchmark", required=True)
        for name, suite in SUITES.items():
            p = bs.add_parser(name)
            suite.add_args(p)
            if cmd == "infer":
                p.add_argument("--output_dir", "--save_dir", dest="output_dir", required=True)
                p.add_argument("--inference_mode", default=suite.modes[0], choices=suite.modes)
                p.add_argument("--base_url", default=None, help="use a served model instead of loading one")
                p.add_argument("--request_timeout", type=float, default=3600.0)
                add_model_args(p)
                add_sampling_args(p)
                p.add_argument("--img_cfg_scale", type=float, default=1.0)
                p.add_argument("--min_pixels", type=int, default=1024 * 1024)
                p.add_argument("--max_pixels", type=int, default=2048 * 2048)
                p.add_argument("--target_image_size", type=square, default=None)
                p.add_argument("--limit", type=int, default=None)
                p.add_argument("--overwrite", action="store_true")
                p.add_argument("--resume", action="store_true", help="accepted: finished samples are always skipped")
                p.add_argument("--num_shards", type=int, default=None)
                p.add_argument("--shard_rank", "--shard_index", dest="shard_rank", type=int, default=None)
                p.add_argument("--workers", type=int, default=1, help="parallel requests (served model)")
            else:
                p.add_argument("--run_dir", "--input_dir", dest="run_dir", required=True)
                p.add_argument("--api_base", "--endpoint", "--api_base_url", dest="api_base", default=None)
                p.add_argument("--api_key", default=None)
                p.add_argument("--judge_model", "--model", dest="judge_model", default=None)
                p.add_argument("--timeout", type=int, default=240)
                p.add_argument("--workers", "--num_workers", dest="workers", type=int, default=16)
                p.add_argument("--force_rerun", "--force", dest="force_rerun", action="store_true")
                p.add_argument("--model_tag", default="model", help="name of the evaluated model in the tables")
    return ap


def main(argv=None, engine=None, client=None):
    a = parser().parse_args(normalise_flags(sys.argv[1:] if argv is None else argv))
    suite = SUITES[a.benchmark]
    return infer(suite, a, engine) if a.cmd == "infer" else score(suite, a, client)


if __name__ == "__main__":
    main()
