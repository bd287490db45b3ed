#!/usr/bin/env python
"""Scores generated pictures with a VLM judge.  One driver covers the three judging styles of the
reference's generation benchmarks:

* ``checklist``  yes/no questions per picture, pass rate per dimension (BizGenEval, IGenBench, TIIF:
  evaluation/gen/bizgeneval/eval_images_bizgeneval.py, evaluation/gen/igenbench/eval_images_igenbench.py,
  evaluation/gen/tiif/eval/eval_with_vlm_mp.py);
* ``text``       the judging model transcribes the text in the picture, compared with the text the prompt asked for
  (CVTG, LongText: evaluation/gen/cvtg/eval_cvtg.py, evaluation/gen/longtext/eval_images_longtext.py);
* ``rating``     a 0-10 rating of prompt following.

Input: the folder written by ``evaluation/generate_for_benchmark.py`` (``metadata.rank*.jsonl`` with
``index``, ``prompt``, ``samples``; pictures at ``<index>/samples/<k>.png``; benchmark fields are copied
from the prompt file: ``questions`` (list of strings) and ``dimension`` for checklists, ``target_texts`` for
text rendering).  A record may also list its pictures itself (``images``: paths relative to the folder).

    python evaluation/gen/judge_images.py --run runs/tiif --mode checklist --workers 16
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from evaluation.common import metrics  # noqa: E402
from evaluation.common.judge import JudgeClient, ResultLog, parse_score, parse_yes_no, run_parallel  # noqa: E402

CHECK_SYSTEM = ("You verify statements about a picture. Answer with 'yes' or 'no' first, then one short sentence "
                "of justification. Judge only what is visible.")
READ_SYSTEM = "You transcribe text in pictures exactly as written, keeping the reading order. Output only the text."
RATE_SYSTEM = ("You rate how well a picture follows its prompt on a scale from 0 (unrelated) to 10 (every detail "
               "right). Answer as 'score: N' followed by one sentence.")


def load_items(run_dir: Path):
    items = []
    for meta in sorted(run_dir.glob("metadata*.jsonl")):
        for line in meta.read_text().splitlines():
            if not line.strip():
                continue
            rec = json.loads(line)
            imgs = rec.get("images") or [f"{rec['index']:05d}/samples/{k:04d}.png" for k in range(rec.get("samples", 1))]
            for k, img in enumerate(imgs):
                items.append({**{a: b for a, b in rec.items() if a != "images"}, "id": f"{rec['index']}/{k}",
                              "image": str(run_dir / img) if not os.path.isabs(img) else img})
    return items


def judge_one(client: JudgeClient, mode: str, it: dict) -> dict:
    if mode == "checklist":
        answers = [client.ask(q, [it["image"]], CHECK_SYSTEM, max_tokens=64) for q in it["questions"]]
        return {"dimension": it.get("dimension", "all"), "checks": [parse_yes_no(a) for a in answers], "answers": answers}
    if mode == "text":
        read = client.ask("Transcribe all text in this picture.", [it["image"]], READ_SYSTEM, max_tokens=1024)
        return {"target_texts": it["target_texts"], "read_text": read}
    ans = client.ask(f"Prompt: {it['prompt']}\nRate the picture.", [it["image"]], RATE_SYSTEM, max_tokens=96)
    return {"dimension": it.get("dimension", "all"), "score": parse_score(ans), "answer": ans}


def summarize(mode: str, records):
    ok = [r for r in records if "error" not in r]
    if mode == "checklist":
        s = metrics.checklist_scores(ok)
    elif mode == "text":
        s = metrics.text_rendering_scores(ok)
    else:
        s = metrics.rating_scores(ok)
    s["errors"] = len(records) - len(ok)
    return s


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--run", required=True, help="folder written by generate_for_benchmark.py")
    ap.add_argument("--mode", required=True, choices=["checklist", "text", "rating"])
    ap.add_argument("--workers", type=int, default=8)
    ap.add_argument("--api_base", default=None)
    ap.add_argument("--model", default=None)
    ap.add_argument("--max_retries", type=int, default=6)
    a = ap.parse_args(argv)
    run = Path(a.run)
    client = JudgeClient(a.api_base, model=a.model, max_retries=a.max_retries)
    log = ResultLog(run / f"judge_{a.mode}.jsonl")
    records = run_parallel(load_items(run), lambda it: judge_one(client, a.mode, it), log, a.workers)
    scores = summarize(a.mode, records)
    (run / f"scores_{a.mode}.json").write_text(json.dumps(scores, indent=1))
    print(metrics.format_table(scores, f"{run.name} [{a.mode}]"))
    return scores


if __name__ == "__main__":
    main()
