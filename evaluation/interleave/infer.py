#!/usr/bin/env python
"""Inference side of the interleaved / visual-reasoning benchmarks (BabyVision, Unimmmu, RealUnify, OpenING;
reference evaluation/interleave/*/infer*.py): every question (text plus optional pictures) goes through
interleaved generation, the answer text and the pictures the model drew on the way are saved.

Questions come from a JSONL (``id``, ``question``, optional ``images`` (paths), ``options``, ``answer``,
``category``).  The model is either served (``--base_url``) or loaded in-process (``--model_path`` /
``--random_init``).  Ranks of a torchrun launch (or ``--shard i/n``) split the file; ``score.py`` merges.

    python evaluation/interleave/infer.py --data babyvision.jsonl --out runs/babyvision --base_url http://127.0.0.1:8000
"""
from __future__ import annotations

import argparse
import base64
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from evaluation.common.judge import ResultLog, run_parallel  # noqa: E402

CHOICE_HINT = "\nAnswer with the option letter, as 'Answer: X'."


def build_question(rec: dict) -> str:
    q = rec["question"]
    if rec.get("options"):
        q += "\n" + "\n".join(f"({chr(65 + i)}) {o}" for i, o in enumerate(rec["options"])) + CHOICE_HINT
    return q


class ServedModel:
    def __init__(self, base_url: str, timeout: float = 3600.0, **gen):
        self.base_url, self.timeout, self.gen = base_url.rstrip("/"), timeout, gen

    def __call__(self, question: str, image_paths):
        import requests
        content = [{"type": "text", "text": question}]
        for p in image_paths:
            b64 = base64.b64encode(Path(p).read_bytes()).decode()
            content.append({"type": "image_url", "image_url": {"url": "data:image/png;base64," + b64}})
        r = requests.post(self.base_url + "/v1/chat/completions", timeout=self.timeout,
                          json={"messages": [{"role": "user", "content": content}], "interleave": True, **self.gen})
        r.raise_for_status()
        msg = r.json()["choices"][0]["message"]["content"]
        if isinstance(msg, str):
            return msg, []
        text = "\n".join(p.get("text", "") for p in msg if p.get("type") == "text")
        pics = [base64.b64decode(p["image_url"]["url"].split(",", 1)[1]) for p in msg if p.get("type") == "image_url"]
        return text, pics


class LocalModel:
    def __init__(self, model_path=None, random_init=None, **gen):
        from sensenova_u1_b200.inference.api import ByteTokenizer, NEOChatModel
        if random_init:
            from sensenova_u1_b200.config import get_config
            cfg = get_config(random_init, **({"head_dim": 128} if random_init == "tiny-mot" else {}))
            self.model, self.tok = NEOChatModel.from_config(cfg), ByteTokenizer(cfg.vocab_size)
        else:
            from transformers import AutoTokenizer
            self.model, self.tok = NEOChatModel.from_pretrained(model_path), AutoTokenizer.from_pretrained(model_path)
        self.gen = gen

    def __call__(self, question: str, image_paths):
        import io
        from PIL import Image
        import numpy as np
        from sensenova_u1_b200.inference.images import load_image_native
        f = self.model.cfg.token_pixels
        imgs = [load_image_native(p, factor=f, normalize="imagenet") for p in image_paths]
        text, pics = self.model.interleave_gen(self.tok, question, imgs, max_rounds=self.gen.get("max_rounds", 4),
                                               max_new_tokens=self.gen.get("max_tokens", 512),
                                               num_steps=self.gen.get("num_steps", 50), seed=self.gen.get("seed", 0))
        out = []
        for p in pics:
            arr = ((p.float().cpu().clamp(-1, 1) + 1) * 127.5).round().byte().permute(1, 2, 0).numpy()
            buf = io.BytesIO()
            Image.fromarray(np.ascontiguousarray(arr), "RGB").save(buf, format="PNG")
            out.append(buf.getvalue())
        return text, out


def run(records, model, out_dir: Path, log: ResultLog, workers: int = 1):
    (out_dir / "images").mkdir(parents=True, exist_ok=True)
    root = Path(records[0].get("_root", ".")) if records else Path(".")

    def one(rec):
        paths = [str((root / p)) if not os.path.isabs(p) else p for p in rec.get("images", [])]
        text, pics = model(build_question(rec), paths)
        names = []
        for k, data in enumerate(pics):
            name = f"images/{str(rec['id']).replace('/', '_')}_{k}.png"
            (out_dir / name).write_bytes(data)
            names.append(name)
        return {"prediction": text, "generated_images": names, "answer": rec.get("answer"),
                "category": rec.get("category", "all"), "options": rec.get("options")}

    return run_parallel(records, one, log, workers)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--base_url", default=None)
    ap.add_argument("--model_path", default=None)
    ap.add_argument("--random_init", default=None)
    ap.add_argument("--shard", default=None, help="i/n: take every n-th question starting at i (default: RANK/WORLD_SIZE)")
    ap.add_argument("--workers", type=int, default=1)
    ap.add_argument("--max_rounds", type=int, default=4)
    ap.add_argument("--max_tokens", type=int, default=512)
    ap.add_argument("--num_steps", type=int, default=50)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    i, n = (int(x) for x in a.shard.split("/")) if a.shard else (int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)))
    root = str(Path(a.data).resolve().parent)
    with open(a.data) as f:
        recs = [dict(json.loads(l), _root=root) for l in f if l.strip()]
    recs = recs[i::n]
    gen = dict(max_rounds=a.max_rounds, max_tokens=a.max_tokens, num_steps=a.num_steps, seed=a.seed)
    model = ServedModel(a.base_url, **gen) if a.base_url else LocalModel(a.model_path, a.random_init, **gen)
    out = Path(a.out)
    log = ResultLog(out / (f"predictions_{i:03d}.jsonl" if n > 1 else "predictions.jsonl"))
    done = run(recs, model, out, log, a.workers)
    print(f"{len(done)} predictions in {log.path}")


if __name__ == "__main__":
    main()
