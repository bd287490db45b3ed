#!/usr/bin/env python
"""Runs the understanding benchmarks (MMMU-Pro, MMLU-Pro, MMBench, AI2D, MathVista, IFEval) with EvalScope against a
served model.  The reference does this with a three-line script over a fixed YAML (evaluation/understanding/es.py,
config.yaml); here the endpoint, the task list and the judge come from flags or the environment, so the same file
serves a laptop and a cluster.

    python -m sensenova_u1_b200.serving.balancer --replicas 8 --model_path CKPT --port 9000 &
    python evaluation/understanding/run_evalscope.py --api_url http://127.0.0.1:9000/v1/ \\
        --judge_api_url https://host/v1 --judge_api_key KEY [--datasets mm_bench ai2d] [--limit 50]

EvalScope is an external package (``pip install evalscope``); without it the script prints the resolved
configuration and stops.  ``evaluation/understanding/run_vqa.py`` is the dependency-free alternative for JSONL
question files."""
import argparse
import json
import os
import sys
from pathlib import Path

import yaml

HERE = Path(__file__).resolve().parent


def resolve_config(a) -> dict:
    cfg = yaml.safe_load((Path(a.config) if a.config else HERE / "evalscope_config.yaml").read_text())
    if a.api_url or os.environ.get("U1_API_URL"):
        cfg["api_url"] = a.api_url or os.environ["U1_API_URL"]
    if a.model:
        cfg["model"] = a.model
    if a.datasets:
        cfg["datasets"] = list(a.datasets)
    if a.limit:
        cfg["limit"] = a.limit
    if a.batch_size:
        cfg["eval_batch_size"] = a.batch_size
    if a.no_thinking:
        cfg["generation_config"]["extra_body"]["chat_template_kwargs"]["enable_thinking"] = False
        cfg["dataset_args"].pop("remove_until", None)
    j = cfg["judge_model_args"]
    j["api_url"] = a.judge_api_url or os.environ.get("JUDGE_API_BASE", j.get("api_url", ""))
    j["api_key"] = a.judge_api_key or os.environ.get("JUDGE_API_KEY", j.get("api_key", ""))
    if a.judge_model:
        j["model_id"] = a.judge_model
    if a.work_dir:
        cfg["work_dir"] = cfg["use_cache"] = a.work_dir
    return cfg


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--config", default=None, help="another YAML in the same schema")
    ap.add_argument("--api_url", default=None)
    ap.add_argument("--model", default=None)
    ap.add_argument("--datasets", nargs="*", default=None)
    ap.add_argument("--limit", type=int, default=None, help="samples per task (smoke runs)")
    ap.add_argument("--batch_size", type=int, default=None)
    ap.add_argument("--no_thinking", action="store_true")
    ap.add_argument("--judge_api_url", default=None)
    ap.add_argument("--judge_api_key", default=None)
    ap.add_argument("--judge_model", default=None)
    ap.add_argument("--work_dir", default=None)
    ap.add_argument("--dry_run", action="store_true", help="print the resolved configuration and stop")
    a = ap.parse_args(argv)
    cfg = resolve_config(a)
    if a.dry_run:
        print(json.dumps(cfg, indent=1))
        return cfg
    try:
        from evalscope import run_task
    except ImportError:
        print(json.dumps(cfg, indent=1))
        print("evalscope is not installed (pip install evalscope); the configuration above is what would run", file=sys.stderr)
        return cfg
    return run_task(task_cfg=cfg)


if __name__ == "__main__":
    main()
