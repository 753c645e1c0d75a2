"""The reference arm of bench.py: 12vivi/tandem itself, unmodified, from ``baseline/_ref``.

``baseline/_ref/tandem`` is the reference's own package folder (``python/tandem`` of its checkout:
what its wheel contains, since its build configuration lists exactly that folder as the wheel's
packages).  This file imports the engine from there and from nowhere else, builds the model of the
benchmark through the reference's ``ModelConfig.from_dict`` + ``build_model`` with seeded
N(0, 0.02) bfloat16 weights made on the device, and drives the reference's ``LLMEngine`` through
its public calls (``add_request``, ``step``, ``generate``) with its stock options, as its own
offline benchmark does (benchmarks/bench_offline.py:45-62 of 12vivi/tandem).  Nothing of
``tandem_b200`` is imported on this path.

The same quantities are measured as for this repository's arm: decode steps of ``--batch`` requests
just behind their 2,048-token prompts (device time by CUDA events and wall-clock time around K
calls of ``engine.step()``), one prefill of 2,048 tokens, and the decode points at batch 1 and 64.
"""

from __future__ import annotations

import os
import sys
import time
import traceback

HERE = os.path.dirname(os.path.abspath(__file__))
REF_ROOT = os.path.join(HERE, "_ref")


def reference_present() -> bool:
    return os.path.isfile(os.path.join(REF_ROOT, "tandem", "engine", "llm_engine.py"))


def _import_reference():
    if REF_ROOT not in sys.path:
        sys.path.insert(0, REF_ROOT)
    import tandem  # noqa: F401

    where = os.path.dirname(os.path.abspath(tandem.__file__))
    if not where.startswith(REF_ROOT):
        raise ImportError(f"'tandem' was imported from {where}, not from baseline/_ref")
    from tandem.config import EngineConfig
    from tandem.engine.llm_engine import LLMEngine
    from tandem.model_config import ModelConfig
    from tandem.models import build_model
    from tandem.sampling_params import SamplingParams

    return EngineConfig, LLMEngine, ModelConfig, build_model, SamplingParams


def _random_model(ModelConfig, build_model, shape: dict, layers: int, max_len: int, seed: int = 0):
    """The reference's own module tree for ``shape``, parameters drawn on the device: matrices
    N(0, 0.02), norm weights one (what this repository's arm draws)."""
    import torch

    mc = ModelConfig.from_dict(dict(shape, num_hidden_layers=layers, max_position_embeddings=max_len))
    torch.manual_seed(seed)
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)  # parameters only: the rotary tables name float32 themselves
    try:
        with torch.device("cuda"):
            model = build_model(mc, max_len)
    finally:
        torch.set_default_dtype(old)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02)
            else:
                p.fill_(1.0)
    return mc, model


def _build(api, shape: dict, layers: int, max_seqs: int, tokens_per_seq: int, backend: str, page: int):
    EngineConfig, LLMEngine, ModelConfig, build_model, _ = api
    max_len = max(4096, -(-tokens_per_seq // page) * page)
    mc, model = _random_model(ModelConfig, build_model, shape, layers, max_len)
    pages = max_seqs * (-(-tokens_per_seq // page)) + 8
    cfg = EngineConfig(model="", device="cuda", dtype="bfloat16", block_size=page, num_kv_blocks=pages,
                       max_num_seqs=max_seqs, max_num_batched_tokens=2048, max_model_len=max_len,
                       attention_backend=backend, cuda_graph_max_bs=max_seqs)
    return LLMEngine(cfg, model_config=mc, model=model, load_tokenizer=False)


def _decode(engine, SamplingParams, prompts: list, steps: int, warmup: int, new_tokens: int) -> dict:
    import torch

    batch = len(prompts)
    sp = SamplingParams(max_tokens=new_tokens + steps + 2 * warmup + 16, temperature=0.0, ignore_eos=True)
    ids = [engine.add_request(p, sp) for p in prompts]
    while engine.scheduler.waiting or any(not r.is_decoding for r in engine.requests.values()):
        engine.step()  # prefill, untimed
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        engine.step()
    stop.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    ms = start.elapsed_time(stop) / steps
    context = max(r.num_computed_tokens for r in engine.requests.values())
    for rid in ids:
        engine.abort_request(rid)
    while engine.has_unfinished_requests():  # the step in flight
        engine.step()
    return dict(ms=ms, tok_s=batch * 1000.0 / ms, e2e_tok_s=batch * steps / wall, e2e_ms=wall * 1000.0 / steps,
                context=context)


def _prefill(engine, SamplingParams, make_prompts, warmup: int, reps: int = 3) -> dict:
    """Wall-clock time of ``generate`` on one fresh 2,048-token prompt with one new token
    (different tokens every time, so the prefix cache has nothing of it)."""
    import torch

    times = []
    for i in range(warmup + reps):
        toks = make_prompts(1, seed=1000 + i)[0]
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        engine.generate([toks], SamplingParams(max_tokens=1, temperature=0.0, ignore_eos=True))
        torch.cuda.synchronize()
        if i >= warmup:
            times.append((time.perf_counter() - t0) * 1000.0)
    ms = sorted(times)[len(times) // 2]
    return dict(ms=ms, tok_s=len(toks) * 1000.0 / ms, tokens=len(toks))


def _measure(args, shapes: dict, make_prompts, clock_sampler, backend: str) -> dict:
    import torch

    api = _import_reference()
    SamplingParams = api[4]
    name, shape = shapes[args.shape]
    layers = args.layers or shape["num_hidden_layers"]
    new_tokens = args.new_tokens or 256
    warmup = max(3, args.warmup)
    page = 16
    max_batch = max(args.batch, 1 if args.no_points else 64)
    per_seq = max(args.prompt_len, 2048) + new_tokens + args.steps + 2 * warmup + 32
    engine = _build(api, shape, layers, max_batch, per_seq, backend, page)
    sampler = clock_sampler()
    sampler.start()
    main_pt = _decode(engine, SamplingParams, make_prompts(args.batch, seed=args.batch, length=args.prompt_len),
                      args.steps, warmup, new_tokens)
    pre = _prefill(engine, SamplingParams, make_prompts, warmup)
    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(_decode(engine, SamplingParams, make_prompts(b, seed=b, length=args.prompt_len),
                                                   args.steps, warmup, new_tokens)["tok_s"], 1)
    clocks = sampler.stop()
    mc = engine.model_config
    return {
        "impl": "reference",
        "metric": f"decode tok/s at batch {args.batch}, {name}, {args.prompt_len:,}-token prompts (one B200)",
        "value": round(main_pt["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(main_pt["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: seeded random weights N(0,0.02) and random token ids",
        "config": {"model": name, "layers": mc.num_hidden_layers, "layers_full": shape["num_hidden_layers"],
                   "hidden": mc.hidden_size, "q_heads": mc.num_attention_heads, "kv_heads": mc.num_key_value_heads,
                   "head_dim": mc.head_dim, "intermediate": mc.intermediate_size, "vocab": mc.vocab_size,
                   "global_batch": args.batch, "seq_len": main_pt["context"], "prompt_len": args.prompt_len,
                   "page_size": page, "parallelism": "single GPU", "backend": engine.backend_name,
                   "cuda_graph": engine.runner.graph_runner is not None, "overlap_schedule": bool(engine.overlap),
                   "gemv_layers": engine.num_gemv_layers, "fused_layers": engine.num_fused_layers},
        "timing": "CUDA events and wall clock around K calls of LLMEngine.step()",
        "e2e": {"value": round(main_pt["e2e_tok_s"], 1), "unit": "tok/s", "ms_per_step": round(main_pt["e2e_ms"], 4),
                "h2d_bytes_per_step": None, "d2h_bytes_per_step": 8 * args.batch},
        "prefill": {"value": round(pre["tok_s"], 1), "tokens": pre["tokens"], "ms": round(pre["ms"], 3),
                    "timing": "wall clock around LLMEngine.generate of one prompt, one new token"},
        "points": points, "clocks": clocks,
        "imports_tandem_b200": any(m == "tandem_b200" or m.startswith("tandem_b200.") for m in sys.modules),
        "torch": torch.__version__,
    }


def _one_line(exc: BaseException) -> str:
    text = f"{type(exc).__name__}: {exc}".strip().splitlines()
    where = traceback.extract_tb(exc.__traceback__)[-1]
    return f"{text[0][:300]} (at {os.path.basename(where.filename)}:{where.lineno})"


def run_reference(args, shapes: dict, make_prompts, clock_sampler) -> dict:
    """The JSON line of the reference arm.  The reference picks its backend itself
    (``attention_backend="auto"``: its FlashInfer path where flashinfer imports, its PyTorch path
    otherwise).  If that stock choice raises on this machine, the error is recorded and the
    reference's other backend option (``"torch"``) is measured instead; only if both raise does the
    arm report itself unavailable, with the errors it met."""
    if not reference_present():
        return {"impl": "reference", "unavailable": "baseline/_ref/tandem is missing: the reference's package folder "
                "(python/tandem of its checkout) has not been placed there"}
    if args.workload != "decode":
        return {"impl": "reference", "unavailable": f"the reference arm measures the decode workload, not {args.workload!r}"}
    import torch

    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device here: the reference arm times 12vivi/tandem on a B200"}
    forced = os.environ.get("TANDEM_REFERENCE_BACKEND")
    errors = []
    for backend in ([forced] if forced else ["auto", "torch"]):
        try:
            out = _measure(args, shapes, make_prompts, clock_sampler, backend)
            if errors:
                out["stock_backend_error"] = errors[0][:300]
            return out
        except Exception as exc:  # a real failure of the reference on this machine: recorded, not hidden
            errors.append(f"attention_backend={backend}: {_one_line(exc)}")
            try:
                import gc

                import torch

                gc.collect()
                torch.cuda.empty_cache()
            except Exception:
                pass
    return {"impl": "reference", "unavailable": "; ".join(errors)[:900]}
