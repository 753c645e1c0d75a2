"""Decode and prefill throughput of the engine on one B200, as one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--impl reference]
                    [--shape 8b|14b|32b] [--prompt-len P] [--new-tokens T] [--workload decode|mixed]

The model has the layer sizes of Qwen3-8B with seeded random weights made on the device; prompts
are seeded random token ids.  A step is one decode step of ``--batch`` requests whose prompts
(2,048 tokens each) were prefilled before the timed region.  ``value`` is decoded tokens per second
timed on the device around K steps of the step function plus the sampling kernel; ``e2e`` is the
same through ``LLMEngine.step()`` with host token ids in and sampled tokens out every step.
Every decode step reads all weights (15 GB, far larger than the 126 MB L2), so nothing is served
from L2 between iterations.  12vivi/tandem measures the same quantities with
benchmarks/bench_offline.py:54-62 (random ids, greedy, ignore_eos).

``--shape`` takes the layer sizes of Qwen3-14B or Qwen3-32B instead (the default line is the one
of Qwen3-8B).  ``--workload mixed`` runs requests with prompts of random lengths (128 to 4,096
tokens) through the scheduler with 128 greedy tokens each, prompt portions of up to 2,048 tokens
beside decoded tokens, and prints its own line: generated and processed tokens per second of
wall-clock time (benchmarks/bench_offline.py:64-86 of 12vivi/tandem).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Qwen3-8B layer sizes (the configuration the benchmark is quoted on)
QWEN3_8B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, hidden_size=4096,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288, vocab_size=151936,
                rope_theta=1000000.0, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=4096)
QWEN3_14B = dict(QWEN3_8B, num_hidden_layers=40, hidden_size=5120, num_attention_heads=40, intermediate_size=17408)
QWEN3_32B = dict(QWEN3_8B, num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, intermediate_size=25600)
SHAPES = {"8b": ("Qwen3-8B shape", QWEN3_8B), "14b": ("Qwen3-14B shape", QWEN3_14B), "32b": ("Qwen3-32B shape", QWEN3_32B)}
PROMPT, NEW_TOKENS, PAGE = 2048, 256, 16


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm_gbs=float(d.get("hbm_gbs", 6650.0)), tflops=float(d.get("bf16_tflops", 1590.0)),
                    tflops_sustained=float(d.get("bf16_tflops_sustained", d.get("bf16_tflops", 1590.0))), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while the timed regions run."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self) -> None:
        self.path = tempfile.mktemp(suffix=".csv")
        self.proc = None

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7 or not f[0].isdigit():
                continue
            sm.append(int(f[0])), mx.append(int(f[1]))
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.remove(self.path)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def build_engine(shape: dict, layers: int, max_seqs: int, tokens_per_seq: int, cuda_graph: bool = True,
                 policy: str = "prefill_first", pages: int = 0):
    from tandem_b200 import EngineConfig, LLMEngine
    from tandem_b200.engine.core import random_model

    max_len = max(4096, -(-tokens_per_seq // PAGE) * PAGE)
    decoder, cfg = random_model(dict(shape, max_position_embeddings=max_len), seed=0, dtype="bfloat16", num_layers=layers)
    pages = pages or max_seqs * (-(-tokens_per_seq // PAGE)) + 8
    eng = LLMEngine(EngineConfig(model="", dtype="bfloat16", block_size=PAGE, num_kv_blocks=pages, max_num_seqs=max_seqs,
                                 max_num_batched_tokens=2048, max_model_len=max_len, schedule_policy=policy,
                                 cuda_graph=cuda_graph, cuda_graph_max_bs=max_seqs),
                    decoder=decoder, model_config=cfg, load_tokenizer=False)
    return eng


def prompts(batch: int, seed: int = 0, length: int = PROMPT) -> list:
    import torch

    g = torch.Generator().manual_seed(seed)
    return [torch.randint(10, 100000, (length,), generator=g).tolist() for _ in range(batch)]


def decode_bytes(eng, batch: int, context: int) -> float:
    """What one decode step has to read: every weight it uses once (the embedding table is only
    gathered from) and the cache of the live requests."""
    from tandem_b200.engine.core import kv_bytes_per_token

    d = eng.decoder
    weights = d.parameter_bytes - d.embedding.numel() * d.embedding.element_size() * (0 if d.head is d.embedding else 1)
    return weights + batch * context * kv_bytes_per_token(d)


def measure_decode(eng, batch: int, steps: int, warmup: int, prompt_len: int = PROMPT, new_tokens: int = NEW_TOKENS) -> dict:
    """Device time of ``steps`` decode steps of ``batch`` requests just behind their prompts of
    ``prompt_len`` tokens, then the same through LLMEngine.step()."""
    import torch

    from tandem_b200 import SamplingParams
    from tandem_b200.kernels import ops

    sp = SamplingParams(max_tokens=new_tokens + steps + 2 * warmup + 16, temperature=0.0, ignore_eos=True)
    for p in prompts(batch, seed=batch, length=prompt_len):
        eng.add_request(p, sp)
    while any(not r.is_decoding for r in eng.requests.values()) or eng.scheduler.waiting:
        eng.step()  # prefill, untimed
    for _ in range(warmup):
        eng.step()
    torch.cuda.synchronize()

    # end to end: host ids in, sampled tokens out, every step
    t0 = time.perf_counter()
    for _ in range(steps):
        eng.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    h2d = eng.executor.h2d_bytes_last  # what one of these steps copied to the device: its batch description
    eng.drain()  # the step in flight (overlap scheduling)

    # device-timed: the step function and the sampling kernel back to back, no host read in between
    plan = eng.scheduler.schedule()
    entries = eng.entries_of(plan)
    for e in entries:
        e.want = [0]
    runner = eng.graphs if (eng.graphs is not None and eng.graphs.takes(entries)) else eng.executor
    context = max(r.num_computed_tokens for r in eng.requests.values())
    for _ in range(max(1, warmup)):
        ops.argmax(runner.run(entries))
    torch.cuda.synchronize()
    before = ops.launches
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        ops.argmax(runner.run(entries))
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / steps
    launches = (ops.launches - before) // steps if eng.graphs is None else eng.graphs.launches_per_replay(entries) + 1
    for rid in list(eng.requests):
        eng.abort_request(rid)
    assert eng.cache.all_free()
    return dict(ms=ms, tok_s=batch * 1000.0 / ms, e2e_tok_s=batch * steps / e2e_s, e2e_ms=e2e_s * 1000 / steps,
                context=context, launches=launches, bytes=decode_bytes(eng, batch, context), h2d=h2d)


def measure_prefill(eng, warmup: int, reps: int = 3) -> dict:
    import torch

    from tandem_b200.engine.executor import StepEntry

    toks = prompts(1, seed=99)[0]
    times = []
    for i in range(warmup + reps):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        eng.executor.step([StepEntry(f"p{i}", toks, [PROMPT - 1])], end=[f"p{i}"])
        stop.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(start.elapsed_time(stop))
    ms = sorted(times)[len(times) // 2]
    c = eng.model_config
    per_layer = c.hidden_size * (c.q_size + 2 * c.kv_size) + c.q_size * c.hidden_size + 3 * c.hidden_size * c.intermediate_size
    linear = 2.0 * PROMPT * c.num_hidden_layers * per_layer + 2.0 * c.hidden_size * c.vocab_size  # one row of logits
    attn = c.num_hidden_layers * 4.0 * c.num_attention_heads * c.head_dim * PROMPT * (PROMPT + 1) / 2
    return dict(ms=ms, tok_s=PROMPT * 1000.0 / ms, flops=linear + attn)


def measure_mixed(eng, num_requests: int, new_tokens: int, seed: int = 0) -> dict:
    """Requests with prompts of random lengths through the scheduler: portions of prompts beside
    decoded tokens, until every request has its ``new_tokens``.  Wall-clock time."""
    import torch

    from tandem_b200 import SamplingParams
    from tandem_b200.kernels import ops

    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(128, 4097, (num_requests,), generator=g).tolist()
    sp = SamplingParams(max_tokens=new_tokens, temperature=0.0, ignore_eos=True)
    result = {}
    for rep in range(2):  # the first pass builds graphs and measures product dispatch; the second is timed
        for n in lengths:
            eng.add_request(torch.randint(10, 100000, (n,), generator=g).tolist(), sp)
        torch.cuda.synchronize()
        before, steps, t0 = ops.launches, 0, time.perf_counter()
        while eng.has_unfinished_requests():
            eng.step()
            steps += 1
        torch.cuda.synchronize()
        seconds = time.perf_counter() - t0
        assert eng.cache.all_free()
        result = dict(seconds=seconds, steps=steps, launches=ops.launches - before, prompt_tokens=sum(lengths),
                      new_tokens=num_requests * new_tokens, preemptions=eng.scheduler.num_preemptions)
    return result


def measure_extras(steps: int, warmup: int) -> dict:
    """The two other workloads the benchmark is quoted on, each with a model of its own, as flat
    keys beside the headline: decode at batch 8 at Qwen3-32B sizes (1,024-token prompts), and 32
    requests with prompts of 128 to 4,096 tokens and 128 new tokens each at Qwen3-14B sizes."""
    import gc

    import torch

    out: dict = {}
    pk = peaks()

    def release():
        gc.collect()
        torch.cuda.empty_cache()

    try:
        t0 = time.perf_counter()
        eng = build_engine(QWEN3_32B, QWEN3_32B["num_hidden_layers"], 8, 1024 + 128 + steps + 2 * warmup + 32)
        r = measure_decode(eng, 8, steps, warmup, 1024, 128)
        out.update({"qwen3_32b_layers": eng.model_config.num_hidden_layers, "qwen3_32b_decode_b8_tok_s": round(r["tok_s"], 1),
                    "qwen3_32b_decode_b8_ms": round(r["ms"], 4), "qwen3_32b_decode_b8_e2e_tok_s": round(r["e2e_tok_s"], 1),
                    "qwen3_32b_decode_b8_hbm_frac": round(r["bytes"] / (r["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
                    "qwen3_32b_seconds": round(time.perf_counter() - t0, 1)})
        del eng
    except Exception as exc:  # the headline stands without it
        out["qwen3_32b_error"] = f"{type(exc).__name__}: {exc}"[:200]
    release()
    try:
        t0 = time.perf_counter()
        eng = build_engine(QWEN3_14B, QWEN3_14B["num_hidden_layers"], 32, 4096 + 128)
        r = measure_mixed(eng, 32, 128)
        out.update({"qwen3_14b_layers": eng.model_config.num_hidden_layers,
                    "qwen3_14b_mixed_generated_tok_s": round(r["new_tokens"] / r["seconds"], 1),
                    "qwen3_14b_mixed_processed_tok_s": round((r["new_tokens"] + r["prompt_tokens"]) / r["seconds"], 1),
                    "qwen3_14b_mixed_seconds": round(r["seconds"], 3), "qwen3_14b_mixed_steps": r["steps"],
                    "qwen3_14b_mixed_preemptions": r["preemptions"], "qwen3_14b_seconds": round(time.perf_counter() - t0, 1)})
        del eng
    except Exception as exc:
        out["qwen3_14b_error"] = f"{type(exc).__name__}: {exc}"[:200]
    release()
    return out


def main_mixed(args, name: str, shape: dict) -> int:
    pk = peaks()
    per_request = 4096 + args.new_tokens
    eng = build_engine(shape, args.layers, args.batch, per_request, not args.no_cuda_graph, policy=args.policy)
    sampler = ClockSampler()
    sampler.start()
    r = measure_mixed(eng, args.batch, args.new_tokens)
    clocks = sampler.stop()
    c = eng.model_config
    out = {
        "metric": f"generated tok/s, {args.batch} requests with prompts of 128-4,096 tokens, {name} (one B200)",
        "value": round(r["new_tokens"] / r["seconds"], 1), "unit": "tok/s", "n_gpus": 1, "steps": r["steps"],
        "processed_tok_s": round((r["new_tokens"] + r["prompt_tokens"]) / r["seconds"], 1), "seconds": round(r["seconds"], 3),
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02) and random token ids",
        "config": {"model": name, "layers": c.num_hidden_layers, "layers_full": shape["num_hidden_layers"],
                   "hidden": c.hidden_size, "q_heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
                   "head_dim": c.head_dim, "intermediate": c.intermediate_size, "vocab": c.vocab_size,
                   "requests": args.batch, "prompt_tokens": r["prompt_tokens"], "new_tokens": r["new_tokens"],
                   "token_budget": 2048, "policy": args.policy, "page_size": PAGE, "preemptions": r["preemptions"],
                   "peaks": pk["source"]},
        "gpu_launches": r["launches"], "clocks": clocks,
    }
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="fewer layers than the shape has (both numbers are reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--no-extra", action="store_true", help="skip the Qwen3-32B decode and Qwen3-14B mixed-workload figures")
    ap.add_argument("--no-cuda-graph", action="store_true")
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES))
    ap.add_argument("--prompt-len", type=int, default=PROMPT, help="prompt length of the decode measurements")
    ap.add_argument("--new-tokens", type=int, default=None)
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed"])
    ap.add_argument("--policy", default="prefill_first", choices=["prefill_first", "decode_first"])
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not measured (use --gpus 1)")
        return 2
    if args.impl == "reference":
        from baseline.reference_arm import run_reference

        print(json.dumps(run_reference(args, SHAPES, prompts, ClockSampler)))
        return 0
    args.warmup = max(3, args.warmup)
    name, shape = SHAPES[args.shape]
    if args.layers is None:
        args.layers = shape["num_hidden_layers"]
    if args.workload == "mixed":
        args.new_tokens = args.new_tokens or 128
        if args.batch == 8:
            args.batch = 32
        return main_mixed(args, name, shape)
    args.new_tokens = args.new_tokens or NEW_TOKENS

    pk = peaks()
    max_batch = max(args.batch, 1 if args.no_points else 64)
    eng = build_engine(shape, args.layers, max_batch,
                       max(args.prompt_len, PROMPT) + args.new_tokens + args.steps + 2 * args.warmup + 32, not args.no_cuda_graph)
    sampler = ClockSampler()
    sampler.start()
    main_pt = measure_decode(eng, args.batch, args.steps, args.warmup, args.prompt_len, args.new_tokens)
    pre = measure_prefill(eng, args.warmup)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(measure_decode(eng, b, args.steps, args.warmup, args.prompt_len,
                                                          args.new_tokens)["tok_s"], 1)
    clocks = sampler.stop()
    c = eng.model_config
    h2d_bytes = main_pt["h2d"]
    extra = {}
    if not args.no_extra and not args.no_points and args.shape == "8b" and args.layers == shape["num_hidden_layers"]:
        del eng  # the other models get the memory
        extra = measure_extras(min(args.steps, 32), args.warmup)
        graphs_on = not args.no_cuda_graph
    else:
        graphs_on = eng.graphs is not None
    achieved = main_pt["bytes"] / (main_pt["ms"] * 1e-3) / 1e9
    out = {
        "metric": f"decode tok/s at batch {args.batch}, {name}, {args.prompt_len:,}-token prompts (one B200)",
        "value": round(main_pt["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_pt["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02) and random token ids",
        "config": {"model": name, "layers": c.num_hidden_layers, "layers_full": shape["num_hidden_layers"],
                   "hidden": c.hidden_size, "q_heads": c.num_attention_heads, "kv_heads": c.num_key_value_heads,
                   "head_dim": c.head_dim, "intermediate": c.intermediate_size, "vocab": c.vocab_size,
                   "global_batch": args.batch, "seq_len": main_pt["context"], "prompt_len": args.prompt_len, "page_size": PAGE,
                   "parallelism": "single GPU", "cuda_graph": graphs_on,
                   "l2": "inputs larger than L2: each step streams every weight", "peaks": pk["source"]},
        "e2e": {"value": round(main_pt["e2e_tok_s"], 1), "unit": "tok/s", "ms_per_step": round(main_pt["e2e_ms"], 4),
                "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4 * (args.batch + 1)},
        "gpu_launches": int(main_pt["launches"]) * args.steps,
        "prefill": {"value": round(pre["tok_s"], 1), "tokens": PROMPT, "ms": round(pre["ms"], 3),
                    "frac": round(pre["flops"] / (pre["ms"] * 1e-3) / (pk["tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks,
    }
    if extra:
        out["extra"] = extra
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
