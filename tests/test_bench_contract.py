"""What bench.py answers: more than one GPU is refused in one line with exit code 2; the reference
arm prints one JSON line, which without a GPU says so and on a GPU carries the reference's numbers."""

import json
import os
import subprocess
import sys

import pytest

from conftest import ROOT


def run(*args, timeout=120):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=timeout)


def reference_placed() -> bool:
    return os.path.isfile(os.path.join(ROOT, "baseline", "_ref", "tandem", "engine", "llm_engine.py"))


def test_more_than_one_gpu_is_refused_in_one_line():
    p = run("--gpus", "2", "--steps", "1", "--warmup", "1")
    assert p.returncode == 2
    assert len(p.stdout.strip().splitlines()) == 1 and "one GPU" in p.stdout


def test_reference_arm_without_a_gpu_says_what_is_missing():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present: the arm measures (see the gpu test)")
    p = run("--impl", "reference", "--gpus", "1")
    assert p.returncode == 0
    lines = p.stdout.strip().splitlines()
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and "value" not in d
    # the only two reasons there can be here: the package folder is not placed, or there is no GPU
    assert ("baseline/_ref/tandem is missing" in d["unavailable"]) != reference_placed()
    assert ("no CUDA device" in d["unavailable"]) == reference_placed()


@pytest.mark.gpu
def test_reference_arm_runs_the_reference_on_the_gpu():
    """Two layers of the benchmark's shape, a few steps: the line must carry numbers measured on
    the reference's own engine (its backend is named), with nothing of this package imported."""
    if not reference_placed():
        pytest.skip("baseline/_ref/tandem is not placed on this machine")
    p = run("--impl", "reference", "--layers", "2", "--steps", "4", "--warmup", "3", "--no-points", timeout=1500)
    assert p.returncode == 0, p.stderr[-2000:]
    d = json.loads(p.stdout.strip().splitlines()[-1])
    assert d["impl"] == "reference"
    assert "unavailable" not in d, d
    assert d["value"] > 0 and d["e2e"]["value"] > 0 and d["prefill"]["value"] > 0
    assert d["config"]["backend"] in ("flashinfer", "torch") and d["config"]["layers"] == 2
    assert d["imports_tandem_b200"] is False
