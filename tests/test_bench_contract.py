"""What bench.py answers without a GPU: more than one GPU is refused in one line with exit code 2,
and the reference arm says in one JSON line why it is unavailable."""

import json
import os
import subprocess
import sys

from conftest import ROOT


def run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_refused_in_one_line():
    p = run("--gpus", "2", "--steps", "1", "--warmup", "1")
    assert p.returncode == 2
    assert len(p.stdout.strip().splitlines()) == 1 and "one GPU" in p.stdout


def test_reference_arm_prints_one_json_line():
    p = run("--impl", "reference", "--gpus", "1")
    assert p.returncode == 0
    lines = p.stdout.strip().splitlines()
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and ("unavailable" in d or "value" in d)
