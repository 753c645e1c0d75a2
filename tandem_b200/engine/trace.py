"""Trace replay: feed given token ids through a model step by step and write logits.

Reads one JSON object per line,
``{"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}``,
runs every line as one step of the engine's own step function (the model, cache manager and
kernels that generation uses), writes the float32 logits at the wanted places to
``<out>/<step>.f32`` ([wanted, vocab], little-endian, entries in order, ``want`` in order) and
prints ``done <step>``.  It samples nothing and keeps no model, cache or loader of its own.

12vivi/tandem has no such tool; its nearest pieces are the direct forward of
tests/test_model_equivalence.py:22-26 and the step trace of python/tandem/executor/step_timer.py:57-68.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

from tandem_b200.cache.manager import cdiv


ROUNDING = 64  # --max-tokens counts every live request rounded up to a multiple of this


def pool_pages(max_tokens: int, page_size: int) -> int:
    """Pages per cache group for ``--max-tokens``: the most tokens live requests hold at any time,
    each request's count rounded up to a multiple of 64, or of the page size where pages are larger.
    Every unit of 64 tokens may belong to another request, so each unit gets whole pages of its
    own: 64 / page_size of them where that divides, ceil(64 / page_size) otherwise (pages of 48
    tokens: two per unit).  With pages of 64 tokens or more a request's count is a multiple of the
    page size already, and the pool is ``max_tokens / page_size`` pages."""
    if page_size >= ROUNDING:
        return max(1, cdiv(max_tokens, page_size))
    return max(1, cdiv(max_tokens, ROUNDING) * cdiv(ROUNDING, page_size))


def replay(model: str, dtype: str, out_dir: str, max_tokens: int, lines, device: str = "cuda:0",
           page_size: int = 16, echo=None) -> int:
    """Run the steps read from ``lines``.  The cache pool holds ``max_tokens`` tokens
    (``pool_pages``), so pages are used again as requests end.  Returns the number of steps run."""
    from tandem_b200.engine.core import build_executor, load_model
    from tandem_b200.engine.executor import StepEntry
    from tandem_b200.kernels import ops

    os.makedirs(out_dir, exist_ok=True)
    decoder, _ = load_model(model, dtype, device)
    executor = build_executor(decoder, page_size=page_size, num_pages=pool_pages(max_tokens, page_size),
                              max_requests=64)
    steps = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        entries = [StepEntry(str(e["id"]), list(e["tokens"]), list(e.get("want", []))) for e in rec.get("entries", [])]
        logits = executor.step(entries, end=[str(r) for r in rec.get("end", [])])
        ops.check_status(executor.device)  # a kernel that gave up a wait or met a missing page: no logits are written
        if logits.shape[0]:
            arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
            tmp = os.path.join(out_dir, f".{rec['step']}.f32.tmp")
            arr.tofile(tmp)
            os.replace(tmp, os.path.join(out_dir, f"{rec['step']}.f32"))
        steps += 1
        if echo is not None:
            echo(f"done {rec['step']}")
    return steps


class TraceWriter:
    """Records the steps an engine launches, as lines this tool replays.

    A step's tokens are noted when the step is launched.  With overlap scheduling the newest
    token of a decoding request is then still on the device; the step is completed once the value
    has arrived (by the next launch, or at ``close``).  A request that lost its pages and is read
    from its start again appears under a new id (``<id>~<n>``); every id ends in the last step
    that carries it.  ``close`` writes the file and returns the ``--max-tokens`` a replay needs."""

    def __init__(self, path: str) -> None:
        self.path = path
        self.records: list = []
        self.open_record = None  # (record, [(entry index, request, position of its last token)]) not complete yet
        self.alias: dict = {}  # request id -> its id in the trace
        self.carried: set = set()  # trace ids that a step has carried
        self.num_steps = 0

    def step(self, plan, entries) -> None:
        self._complete()
        record = {"step": self.num_steps, "entries": [], "end": []}
        unknown = []
        for i, (s, e) in enumerate(zip(plan.scheduled, entries)):
            rid = self.alias.setdefault(e.request_id, e.request_id)
            if s.request.num_computed_tokens == 0 and rid in self.carried:  # read from its start again
                rid = self.alias[e.request_id] = f"{e.request_id}~{s.request.num_preemptions}"
            self.carried.add(rid)
            record["entries"].append({"id": rid, "tokens": list(e.tokens), "want": list(e.want)})
            if e.pending is not None:
                unknown.append((i, s.request, s.request.num_computed_tokens + s.num_tokens - 1))
        self.num_steps += 1
        self.open_record = (record, unknown)
        self._complete()

    def _complete(self, final: bool = False) -> None:
        if self.open_record is None:
            return
        record, unknown = self.open_record
        if not final and any(position >= req.num_known for _, req, position in unknown):
            return  # a value is still on its way
        dropped = set()
        for i, req, position in unknown:
            if position < req.num_known:
                record["entries"][i]["tokens"][-1] = req.token_ids[position]
            else:
                dropped.add(i)  # the request ended with this step in flight: the token never reached the host
        record["entries"] = [e for i, e in enumerate(record["entries"]) if i not in dropped]
        self.records.append(record)
        self.open_record = None

    def close(self) -> int:
        self._complete(final=True)
        last = {}
        for index, record in enumerate(self.records):
            for e in record["entries"]:
                last[e["id"]] = index
        for rid, index in last.items():
            self.records[index]["end"].append(rid)
        held, peak = {}, 0
        with open(self.path, "w", encoding="utf-8") as f:
            for record in self.records:
                for e in record["entries"]:
                    held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
                peak = max(peak, sum(cdiv(n, ROUNDING) * ROUNDING for n in held.values()))
                for rid in record["end"]:
                    held.pop(rid, None)
                f.write(json.dumps(record) + "\n")
        return peak


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="trace_run", description="replay a trace of steps and write logits")
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True, help="tokens the cache pool holds")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    args = p.parse_args(argv)

    def echo(text: str) -> None:
        sys.stdout.write(text + "\n")
        sys.stdout.flush()

    replay(args.model, args.dtype, args.out, args.max_tokens, sys.stdin, args.device, args.block_size, echo)
    return 0
