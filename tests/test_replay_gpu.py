"""Replay on the GPU: the same requests whole, with the last 32 tokens one by one, in portions of
changing size, and mixed with other requests in a pool so small that pages are used again; in
true float32 and in bfloat16; all compared with the plain implementation."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import replay_cases as rc
from conftest import PAGE, ROOT, TINY, random_tokens

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 33, 70, 1, 41], "B": [1, 9, 40, 70, 130, 23], "C": [50, 3, 97, 64, 30, 75]}
BUILDERS = {"whole": rc.whole, "tail": rc.tail_one_by_one, "portions": rc.changing_portions, "mixed": rc.mixed}


def requests_of(name):
    vocab = TINY[name]["vocab_size"]
    return {f"r{i}": random_tokens(100 * ord(name) + i, n, vocab) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def oracle(tiny_folder):
    """name -> {request id: float64 logits [T, V] of the plain implementation}, and a bfloat16 run of it."""
    cache = {}

    def get(name):
        if name not in cache:
            folder = tiny_folder(name)
            cfg, w64 = plain.read_folder(folder, torch.float64)
            _, w16 = plain.read_folder(folder, torch.bfloat16)
            reqs = requests_of(name)
            full = {rid: plain.forward(cfg, w64, t, torch.float64) for rid, t in reqs.items()}
            low = {rid: plain.forward(cfg, w16, t, torch.bfloat16).double() for rid, t in reqs.items()}
            cache[name] = (full, low)
        return cache[name]

    return get


def run_in_process(folder, dtype, steps, page_size, max_tokens, log=None):
    from tandem_b200.engine.core import build_executor, load_model
    from tandem_b200.engine.executor import StepEntry

    decoder, _ = load_model(folder, dtype, "cuda:0")
    ex = build_executor(decoder, page_size=page_size, num_pages=-(-max_tokens // page_size), max_requests=8)
    pages = rc.PageLog(ex.manager)
    out = {}
    for st in steps:
        logits = ex.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in st["entries"]], end=st["end"])
        if logits.shape[0]:
            out[st["step"]] = logits.cpu().double().numpy()
        ex.manager.check()
    assert ex.manager.all_free()
    if log is not None:
        log.append(pages)
    return out


def check(name, dtype, per_request, oracle):
    full, low = oracle(name)
    for rid, ref in full.items():
        got = torch.from_numpy(np.stack(per_request[rid]))
        assert got.shape == ref.shape, (rid, got.shape, ref.shape)
        err = (got - ref).abs().max().item()
        if dtype == "float32":
            assert err < 1e-4, (name, rid, err, int((got - ref).abs().max(-1).values.argmax()))
        else:
            # the rule of the reference's own GPU test (tests/test_gpu_fastpath.py:107-122): no worse
            # than 1.5 x the error of the same model run plainly in bfloat16, plus 0.02
            base = (low[rid] - ref).abs().max().item()
            assert err <= 1.5 * base + 0.02, (name, rid, err, base, int((got - ref).abs().max(-1).values.argmax()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("regime", list(BUILDERS))
def test_replay_regimes(tiny_folder, oracle, name, dtype, regime):
    reqs = requests_of(name)
    steps = BUILDERS[regime](reqs)
    assert sum(len(e["tokens"]) for s in steps for e in s["entries"]) == sum(len(t) for t in reqs.values())
    if regime == "portions":
        assert any(len(e["tokens"]) == 2 for s in steps for e in s["entries"])
    if regime == "mixed":
        assert max(len(s["entries"]) for s in steps) == 4
        assert any(len({len(e["tokens"]) == 1 for e in s["entries"]}) == 2 for s in steps)  # portions beside single tokens
    need = rc.tokens_needed(steps, round_to=PAGE[name])  # whole pages of this pool, nothing to spare
    log = []
    out = run_in_process(tiny_folder(name), dtype, steps, PAGE[name], need, log)
    assert log[0].pages_reused > 0, "no page was handed out twice: the pool is too large for this trace"
    if regime == "mixed":  # pages that a finished request gave back are written while other requests are read
        assert log[0].reused_beside_live >= 3, log[0].reused_beside_live
    check(name, dtype, rc.collect(steps, out), oracle)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_float32_is_bitwise_the_same_however_it_is_cut(tiny_folder, dtype):
    """In float32 every kernel sums in one fixed order per token, so cutting and batching change
    nothing at all; in bfloat16 they may change the rounding only."""
    reqs = requests_of("B")
    runs = {}
    for regime in ("whole", "portions", "mixed"):
        steps = BUILDERS[regime](reqs)
        log = []
        out = run_in_process(tiny_folder("B"), dtype, steps, PAGE["B"], rc.tokens_needed(steps, round_to=PAGE["B"]), log)
        assert log[0].pages_reused > 0
        runs[regime] = {rid: np.stack(rows) for rid, rows in rc.collect(steps, out).items()}
    for rid in reqs:
        for regime in ("portions", "mixed"):
            diff = np.abs(runs[regime][rid] - runs["whole"][rid]).max()
            assert diff == 0.0 if dtype == "float32" else diff < 0.05, (rid, regime, diff)


MANY = [30, 9, 61, 17, 2, 44, 58, 25, 12, 63, 37, 5, 50, 21]  # 14 requests: four live hold 256 of their 434 tokens at most


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,block_size", [("B", 8), ("A", 16), ("B", 48)])
def test_trace_run_program(tiny_folder, tmp_path, name, block_size, dtype):
    """The program itself, as a user runs it: steps on stdin, ``done <step>`` lines, .f32 files,
    ``--max-tokens`` as the tool defines it (every live request rounded up to 64 tokens); so many
    short requests that the pool's pages go round more than once."""
    from tandem_b200.engine.trace import pool_pages

    vocab = TINY[name]["vocab_size"]
    reqs = {f"m{i}": random_tokens(977 * ord(name) + i, n, vocab) for i, n in enumerate(MANY)}
    steps = rc.mixed(reqs)
    need = rc.tokens_needed(steps, round_to=max(64, block_size))
    twice, beside_live = rc.pages_handed_twice(steps, block_size, pool_pages(need, block_size))
    assert twice >= 3 and beside_live >= 3, (twice, beside_live)
    out_dir = tmp_path / "out"
    proc = subprocess.Popen([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", tiny_folder(name), "--dtype", dtype,
                             "--out", str(out_dir), "--max-tokens", str(need), "--block-size", str(block_size)],
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    for st in steps:  # the next step goes in only after the last one's "done"
        proc.stdin.write(json.dumps(st) + "\n")
        proc.stdin.flush()
        assert proc.stdout.readline().strip() == f"done {st['step']}"
    proc.stdin.close()
    assert proc.wait(timeout=120) == 0
    outputs = {}
    for st in steps:
        wanted = sum(len(e["want"]) for e in st["entries"])
        path = out_dir / f"{st['step']}.f32"
        if wanted:
            outputs[st["step"]] = np.fromfile(path, dtype="<f4").reshape(wanted, vocab).astype(np.float64)
        else:
            assert not path.exists()
    folder = tiny_folder(name)
    cfg, w64 = plain.read_folder(folder, torch.float64)
    _, w16 = plain.read_folder(folder, torch.bfloat16)
    got = rc.collect(steps, outputs)
    for rid, toks in reqs.items():
        ref = plain.forward(cfg, w64, toks, torch.float64)
        err = (torch.from_numpy(np.stack(got[rid])) - ref).abs().max().item()
        if dtype == "float32":
            assert err < 1e-4, (rid, err)
        else:
            base = (plain.forward(cfg, w16, toks, torch.bfloat16).double() - ref).abs().max().item()
            assert err <= 1.5 * base + 0.02, (rid, err, base)


def test_out_of_pages_is_refused_before_anything_runs(tiny_folder):
    from tandem_b200.cache.pages import OutOfPages
    from tandem_b200.engine.core import build_executor, load_model
    from tandem_b200.engine.executor import StepEntry

    decoder, _ = load_model(tiny_folder("A"), "float32", "cuda:0")
    ex = build_executor(decoder, page_size=4, num_pages=4, max_requests=4)
    ex.step([StepEntry("a", list(range(10)), [9])])
    with pytest.raises(OutOfPages):
        ex.step([StepEntry("b", list(range(9)), [8])])
    assert not ex.manager.has("b") and ex.manager.num_tokens("a") == 10
    ex.step([StepEntry("a", [1, 2], [1])], end=["a"])
    assert ex.manager.all_free()
    with pytest.raises(ValueError, match="vocabulary"):
        ex.step([StepEntry("c", [512], [0])])
