#!/usr/bin/env python
"""Scores a file of judged records with one benchmark's rules.

    python -m evaluation.benchmarks.score --benchmark bizgeneval --records runs/biz/judged.jsonl --out runs/biz/summary.json
    python -m evaluation.benchmarks.score --benchmark longtext --mode zh --records runs/lt/judged.jsonl
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


def main(argv=None):
    from . import SCORERS
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--benchmark", required=True, choices=sorted(SCORERS))
    ap.add_argument("--records", required=True, help="judged records (.jsonl, or .json holding a list)")
    ap.add_argument("--mode", default="en", choices=["en", "zh"], help="language of the LongText split")
    ap.add_argument("--out", default=None)
    a = ap.parse_args(argv)
    recs = load_records(a.records)
    summary = SCORERS[a.benchmark](recs, a.mode) if a.benchmark == "longtext" else SCORERS[a.benchmark](recs)
    text = json.dumps(summary, ensure_ascii=False, indent=2)
    if a.out:
        Path(a.out).write_text(text, encoding="utf-8")
    print(text)
    return 0


if __name__ == "__main__":
    sys.exit(main())
