"""Every documented command line builds its parser and prints its help on a machine without a GPU."""
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
COMMANDS = [
    ["-m", "sensenova_u1_b200.train.convert", "--help"],
    ["-m", "sensenova_u1_b200.train.convert", "to-train", "--help"],
    ["-m", "sensenova_u1_b200.serving.balancer", "--help"],
    ["-m", "sensenova_u1_b200.serving.server", "--help"],
    ["-m", "sensenova_u1_b200.utils.param_count", "--help"],
    ["-m", "sensenova_u1_b200.u1_5.briefs", "--help"],
    ["-m", "evaluation.benchmarks.score", "--help"],
    ["evaluation/gen/run_benchmark.py", "generate", "tiif", "--help"],
    ["evaluation/gen/run_benchmark.py", "evaluate", "bizgeneval", "--help"],
    ["evaluation/interleave/run_benchmark.py", "infer", "opening", "--help"],
    ["evaluation/interleave/run_benchmark.py", "score", "realunify_ueg", "--help"],
    ["evaluation/understanding/run_evalscope.py", "--help"],
    ["evaluation/generate_for_benchmark.py", "--help"],
    ["evaluation/gen/judge_images.py", "--help"],
    ["examples/t2i/inference.py", "--help"],
    ["examples/editing/inference.py", "--help"],
    ["examples/interleave/inference.py", "--help"],
    ["examples/vqa/inference.py", "--help"],
    ["examples/serving/client.py", "--help"],
    ["train_sensenovau1.py", "--help"],
    ["bench.py", "--help"],
    ["render_requirements.py", "--help"],
]


@pytest.mark.parametrize("cmd", COMMANDS, ids=lambda c: " ".join(c[:-1]))
def test_help(cmd):
    r = subprocess.run([sys.executable, *cmd], cwd=ROOT, capture_output=True, text=True, timeout=180)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "usage" in r.stdout.lower()
