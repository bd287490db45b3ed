"""Per-benchmark scoring rules of the generation and interleaved benchmarks the reference ships drivers for
(evaluation/gen/{bizgeneval,cvtg,igenbench,longtext,tiif}, evaluation/interleave/{BabyVision,OpenING,Realunify,
Unimmmu}).  Each function takes the judged records written by ``evaluation/gen/judge_images.py`` /
``evaluation/interleave/infer.py`` (plain dicts) and returns the benchmark's summary dict; ``SCORERS`` maps the
benchmark name to its function, ``python -m evaluation.benchmarks.score --benchmark NAME --records FILE`` is the CLI."""
from .rules import (SCORERS, babyvision_summary, bizgeneval_summary, cvtg_summary, igenbench_summary,  # noqa: F401
                    longtext_summary, opening_summary, realunify_summary, tiif_summary, unimmmu_summary)
