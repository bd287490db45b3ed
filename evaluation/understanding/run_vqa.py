#!/usr/bin/env python
"""Visual-understanding benchmarks against a served model: multiple choice (MMMU / MMBench style), short
answers (relaxed match, ChartQA style) and document answers (ANLS, DocVQA style).  The reference runs these
through external harnesses configured for its served endpoint (evaluation/understanding/es.py,
evaluation/easi/config/sensenova_models.py); this driver talks to the same OpenAI-style route directly.

Data: JSONL with ``id``, ``question``, ``images`` (paths), ``answer`` (string or list), optional ``options``,
``category``, ``metric`` (``choice`` | ``relaxed`` | ``anls`` | ``exact``; default by the presence of options).

    python evaluation/understanding/run_vqa.py --data mmmu_val.jsonl --out runs/mmmu --base_url http://127.0.0.1:8000
"""
from __future__ import annotations

import argparse
import base64
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from evaluation.common import metrics  # noqa: E402
from evaluation.common.judge import JudgeClient, ResultLog, parse_choice, run_parallel  # noqa: E402

SHORT_HINT = "\nAnswer with a single word or phrase."
CHOICE_HINT = "\nAnswer with the option letter, as 'Answer: X'."


def score(rec: dict, prediction: str) -> float:
    answers = rec["answer"] if isinstance(rec["answer"], list) else [str(rec["answer"])]
    metric = rec.get("metric") or ("choice" if rec.get("options") else "relaxed")
    if metric == "choice":
        letters = "ABCDEFGHIJ"[: len(rec["options"])]
        return float(parse_choice(prediction, letters) == answers[0].strip().upper())
    if metric == "anls":
        return metrics.anls(prediction, answers)
    if metric == "exact":
        return metrics.exact_match(prediction, answers)
    return metrics.relaxed_match(prediction, answers)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--base_url", default="http://127.0.0.1:8000")
    ap.add_argument("--model", default="sensenova-u1")
    ap.add_argument("--workers", type=int, default=8)
    ap.add_argument("--max_tokens", type=int, default=256)
    a = ap.parse_args(argv)
    root = Path(a.data).resolve().parent
    with open(a.data) as f:
        recs = [json.loads(l) for l in f if l.strip()]
    client = JudgeClient(a.base_url, model=a.model)        # same protocol: a chat endpoint that sees pictures
    log = ResultLog(Path(a.out) / "predictions.jsonl")

    def one(rec):
        q = rec["question"]
        if rec.get("options"):
            q += "\n" + "\n".join(f"({chr(65 + i)}) {o}" for i, o in enumerate(rec["options"])) + CHOICE_HINT
        else:
            q += SHORT_HINT
        imgs = [str(root / p) if not os.path.isabs(p) else p for p in rec.get("images", [])]
        pred = client.ask(q, imgs, max_tokens=a.max_tokens)
        return {"prediction": pred, "correct": score(rec, pred), "category": rec.get("category", "all")}

    done = run_parallel(recs, one, log, a.workers)
    scores = metrics.accuracy_by_category(r for r in done if "error" not in r)
    scores["errors"] = sum(1 for r in done if "error" in r)
    (Path(a.out) / "scores.json").write_text(json.dumps(scores, indent=1))
    print(metrics.format_table(scores, Path(a.out).name))
    return scores


if __name__ == "__main__":
    main()
