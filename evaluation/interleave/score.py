#!/usr/bin/env python
"""Scores the predictions of ``infer.py``: option letters or short answers against the key, overall and per
category (reference evaluation/interleave/BabyVision/compute_score.py, Unimmmu/calculate_score.py,
Realunify/calculate_score.py, plus the ``merge_shards.py`` helpers); open-ended answers can instead be rated by
a judge (OpenING style, reference evaluation/interleave/OpenING/eval_opening.py + summarize_GPT_scores.py).

    python evaluation/interleave/score.py --run runs/babyvision
    python evaluation/interleave/score.py --run runs/opening --judge --workers 8
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from evaluation.common import metrics  # noqa: E402
from evaluation.common.judge import (JudgeClient, ResultLog, merge_shards, parse_choice, parse_score,  # noqa: E402
                                     run_parallel)

RATE_SYSTEM = ("You grade an answer that mixes text and pictures against the task. Consider correctness, "
               "completeness and whether the pictures support the text. Answer as 'score: N' (0-10) and one sentence.")


def is_correct(rec: dict):
    if rec.get("answer") in (None, "") or "error" in rec:
        return None
    if rec.get("options"):
        letters = "ABCDEFGHIJ"[: len(rec["options"])]
        got = parse_choice(rec.get("prediction", ""), letters)
        want = str(rec["answer"]).strip()
        if len(want) != 1 or want.upper() not in letters:       # the key holds the option text, not its letter
            opts = [metrics.normalize_text(o) for o in rec["options"]]
            nw = metrics.normalize_text(want)
            want = letters[opts.index(nw)] if nw in opts else want
        return float(got is not None and got == want.upper())
    answers = rec["answer"] if isinstance(rec["answer"], list) else [str(rec["answer"])]
    tail = rec.get("prediction", "").strip().splitlines()[-1:] or [""]
    return max(metrics.relaxed_match(tail[0], answers), metrics.exact_match(rec.get("prediction", ""), answers))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--run", required=True)
    ap.add_argument("--judge", action="store_true", help="rate open-ended answers with the judging endpoint")
    ap.add_argument("--workers", type=int, default=8)
    a = ap.parse_args(argv)
    run = Path(a.run)
    shards = sorted(glob.glob(str(run / "predictions_*.jsonl")))
    if shards:
        merge_shards(shards, run / "predictions.jsonl")
    recs = ResultLog(run / "predictions.jsonl").records()
    if a.judge:
        client = JudgeClient()
        log = ResultLog(run / "judge_ratings.jsonl")

        def rate(rec):
            imgs = [str(run / p) for p in rec.get("generated_images", [])][:4]
            ans = client.ask(f"Task: {rec.get('question', '')}\nAnswer text: {rec.get('prediction', '')}", imgs,
                             RATE_SYSTEM, max_tokens=96)
            return {"dimension": rec.get("category", "all"), "score": parse_score(ans), "answer": ans}

        scores = metrics.rating_scores(r for r in run_parallel(recs, rate, log, a.workers) if "error" not in r)
    else:
        for r in recs:
            r["correct"] = is_correct(r)
        scores = metrics.accuracy_by_category(recs)
        scores["unanswerable_or_failed"] = sum(1 for r in recs if r["correct"] is None)
    (run / "scores.json").write_text(json.dumps(scores, indent=1))
    print(metrics.format_table(scores, run.name))
    return scores


if __name__ == "__main__":
    main()
