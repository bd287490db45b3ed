#!/usr/bin/env python
"""Scores a file of judged records with one benchmark's rules.

    python -m evaluation.benchmarks.score --benchmark bizgeneval --records runs/biz/judged.jsonl --out runs/biz/summary.json
    python -m evaluation.benchmarks.score --benchmark longtext --mode zh --records runs/lt/judged.jsonl
    python -m evaluation.benchmarks.score --benchmark babyvision --records run1.jsonl run2.jsonl run3.jsonl    # mean +- std

Several record files are scored one by one and every numeric entry of the summaries is reported as mean and standard
deviation over the runs (the reference's BabyVision scorer averages repeated runs this way,
evaluation/interleave/BabyVision/compute_score.py:44-95).
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def load_records(path: str):
    p = Path(path)
    text = p.read_text(encoding="utf-8")
    if p.suffix == ".jsonl":
        return [json.loads(line) for line in text.splitlines() if line.strip()]
    data = json.loads(text)
    return data if isinstance(data, list) else data.get("records", [data])


def across_runs(summaries):
    """Mean and population standard deviation of every number that all summaries share, keeping their nesting."""
    first = summaries[0]
    if isinstance(first, dict):
        keys = [k for k in first if all(isinstance(s, dict) and k in s for s in summaries)]
        out = {k: across_runs([s[k] for s in summaries]) for k in keys}
        return {k: v for k, v in out.items() if v is not None}
    if isinstance(first, bool) or not isinstance(first, (int, float)):
        return None
    vals = [float(s) for s in summaries]
    m = sum(vals) / len(vals)
    return {"mean": m, "std": (sum((v - m) ** 2 for v in vals) / len(vals)) ** 0.5}


def main(argv=None):
    from . import SCORERS
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--benchmark", required=True, choices=sorted(SCORERS))
    ap.add_argument("--records", required=True, nargs="+", help="judged records (.jsonl, or .json holding a list); several "
                                                                "files: repeated runs, reported as mean and std")
    ap.add_argument("--mode", default="en", choices=["en", "zh"], help="language of the LongText split")
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    one = lambda recs: SCORERS[a.benchmark](recs, a.mode) if a.benchmark == "longtext" else SCORERS[a.benchmark](recs)
    runs = [one(load_records(f)) for f in a.records]
    summary = runs[0] if len(runs) == 1 else {"benchmark": a.benchmark, "runs": len(runs), "across_runs": across_runs(runs),
                                              "per_run": runs}
    text = json.dumps(summary, ensure_ascii=False, indent=2)
    if a.out:
        Path(a.out).write_text(text, encoding="utf-8")
    print(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
