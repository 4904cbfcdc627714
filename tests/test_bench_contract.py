"""What bench.py promises without a GPU: more than one GPU is refused with one line and exit code 2,
and the reference arm answers with one JSON line that says why it is unavailable and exits 0."""
from __future__ import annotations

import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], stdout=subprocess.PIPE,
                          stderr=subprocess.PIPE, text=True, timeout=120)


def test_more_than_one_gpu_is_refused_in_one_line():
    done = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert done.returncode == 2
    lines = [line for line in done.stdout.splitlines() if line.strip()]
    assert len(lines) == 1 and "--gpus 2" in lines[0]


def test_reference_arm_says_why_it_is_unavailable():
    done = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert done.returncode == 0
    lines = [line for line in done.stdout.splitlines() if line.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and isinstance(line["unavailable"], str) and line["unavailable"]
