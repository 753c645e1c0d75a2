"""Kernel microbenchmarks: one kernel at a time, on shapes given on the command line.

    python -m tandem_b200.kernels.microbench gemm --m 8 --n 24576 --k 4096
    python -m tandem_b200.kernels.microbench decode-attention --batch 64 --context 2048
    python -m tandem_b200.kernels.microbench prefill-attention --tokens 2048
    python -m tandem_b200.kernels.microbench tokenwise --tokens 2048
    python -m tandem_b200.kernels.microbench norm-gemm --m 8 --n 6144 --k 4096
    python -m tandem_b200.kernels.microbench dispatch [--shapes 8b|14b|32b]
    python -m tandem_b200.kernels.microbench step-timeline --batch 8 --layers 4

Timing follows 12vivi/tandem's kernel benchmarks (benchmarks/bench_gemv.py:3-6,35-56): the calls are
captured in one CUDA graph so that launch cost does not count, and weights or caches are rotated
through copies that together exceed L2, so every call streams from HBM.  ``--no-graph --iters N``
runs N plain launches instead (what a profiler is pointed at).
"""

from __future__ import annotations

import argparse
import math

import torch

L2_BYTES = 126 << 20


def time_calls(fn, iters: int, graph: bool) -> float:
    """Microseconds per call of fn(i), i = 0 .. iters-1."""
    for i in range(min(3, iters)):
        fn(i)
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        start.record()
        g.replay()
        stop.record()
    else:
        start.record()
        for i in range(iters):
            fn(i)
        stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / iters * 1000.0


def copies_for(nbytes: int) -> int:
    return max(2, 3 * L2_BYTES // max(1, nbytes) + 1)


def bench_gemm(args) -> None:
    from tandem_b200.kernels import gemm_bf16

    M, N, K = args.m, args.n, args.k
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies_for(N * K * 2))]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    out = torch.float32 if args.f32_out else torch.bfloat16
    rows = []
    if gemm_bf16.skinny_applies(M, N, K) and args.impl in ("both", "skinny"):
        rows.append(("tcgen05 skinny kernel", time_calls(lambda i: gemm_bf16.skinny(x, ws[i % len(ws)], out), args.iters, args.graph)))
    if gemm_bf16.gemv_applies(M, N, K) and args.impl in ("both", "gemv"):
        rows.append(("mma.sync streaming kernel", time_calls(lambda i: gemm_bf16.gemv(x, ws[i % len(ws)], out), args.iters, args.graph)))
    if args.impl in ("both", "wide") and M > gemm_bf16.SKINNY_MAX_ROWS and gemm_bf16.wide_applies(M, N, K):
        rows.append(("tcgen05 wide kernel", time_calls(lambda i: gemm_bf16.wide(x, ws[i % len(ws)], out), args.iters, args.graph)))
    if args.impl in ("both", "pair") and M > gemm_bf16.SKINNY_MAX_ROWS and gemm_bf16.wide_applies(M, N, K):
        rows.append(("tcgen05 pair kernel", time_calls(lambda i: gemm_bf16.wide_pair(x, ws[i % len(ws)], out), args.iters, args.graph)))
    if args.impl in ("both", "library"):
        rows.append(("library (cuBLAS)", time_calls(lambda i: gemm_bf16._library(x, ws[i % len(ws)], out), args.iters, args.graph)))
    if args.gated and M > gemm_bf16.SKINNY_MAX_ROWS:
        from tandem_b200.kernels import ops

        rows.append(("wide kernel, silu*up fused", time_calls(lambda i: gemm_bf16.wide(x, ws[i % len(ws)], out, gated=True), args.iters, args.graph)))
        rows.append(("pair kernel, silu*up fused", time_calls(lambda i: gemm_bf16.wide_pair(x, ws[i % len(ws)], out, gated=True), args.iters, args.graph)))
        rows.append(("library + silu_mul kernel", time_calls(lambda i: ops.silu_mul(gemm_bf16._library(x, ws[i % len(ws)], out)), args.iters, args.graph)))
    for name, us in rows:
        print(f"gemm M={M} N={N} K={K}  {name:24s} {us:8.1f} us  {N * K * 2 / us / 1e3:7.0f} GB/s weights  "
              f"{2.0 * M * N * K / us / 1e6:7.1f} TFLOP/s")


def bench_norm_gemm(args) -> None:
    """add_rmsnorm followed by the matrix product that reads its output, as a block runs them
    (TANDEM_PDL=0 shows what the programmatic dependent launch between the two is worth)."""
    from tandem_b200.kernels import gemm_bf16, ops

    M, N, K = args.m, args.n, args.k
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies_for(N * K * 2))]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    res, w = torch.randn(M, K, device="cuda"), torch.ones(K, device="cuda")
    for impl, gemm in (("tcgen05 skinny kernel", gemm_bf16.skinny), ("library (cuBLAS)", gemm_bf16._library)):
        if impl.startswith("tcgen05") and not gemm_bf16.skinny_applies(M, N, K):
            continue

        def step(i):
            gemm(ops.add_rmsnorm(x, res, w, 1e-6, torch.bfloat16), ws[i % len(ws)], torch.bfloat16)

        alone = time_calls(lambda i: gemm(x, ws[i % len(ws)], torch.bfloat16), args.iters, args.graph)
        norm = time_calls(lambda i: ops.add_rmsnorm(x, res, w, 1e-6, torch.bfloat16), args.iters, args.graph)
        both = time_calls(step, args.iters, args.graph)
        print(f"norm + gemm M={M} N={N} K={K}  {impl:24s} {both:8.1f} us  (alone: gemm {alone:.1f} us, norm {norm:.1f} us)")


LAYER_SHAPES = {  # (name, N, K) of the products of a layer and the output head
    "8b": [("qkv", 6144, 4096), ("o", 4096, 4096), ("gate_up", 24576, 4096), ("down", 4096, 12288), ("head", 151936, 4096)],
    "14b": [("qkv", 7168, 5120), ("o", 5120, 5120), ("gate_up", 34816, 5120), ("down", 5120, 17408), ("head", 151936, 5120)],
    "32b": [("qkv", 10240, 5120), ("o", 5120, 8192), ("gate_up", 51200, 5120), ("down", 5120, 25600), ("head", 151936, 5120)],
}


def bench_dispatch(args) -> None:
    """Every kernel that takes a shape, timed on the products of a layer at each class of rows, next
    to what the fixed rule of ``gemm_bf16.choose`` picks: the table its thresholds are read off."""
    from tandem_b200.kernels import gemm_bf16, ops

    bf = torch.bfloat16
    for name, N, K in LAYER_SHAPES[args.shapes]:
        ws = [torch.randn(N, K, device="cuda", dtype=bf) * 0.02 for _ in range(copies_for(N * K * 2))]
        out = torch.float32 if name == "head" else bf
        winners = {}
        for M in gemm_bf16.ROW_CLASSES:
            x = torch.randn(M, K, device="cuda", dtype=bf)
            times = {"library": time_calls(lambda i: gemm_bf16._library(x, ws[i % len(ws)], out), args.iters, args.graph)}
            if gemm_bf16.skinny_applies(M, N, K):
                times["skinny"] = time_calls(lambda i: gemm_bf16.skinny(x, ws[i % len(ws)], out), args.iters, args.graph)
            if gemm_bf16.gemv_applies(M, N, K):
                times["gemv"] = time_calls(lambda i: gemm_bf16.gemv(x, ws[i % len(ws)], out), args.iters, args.graph)
            rule, best = gemm_bf16.choose(M, N, K), min(times, key=times.get)
            # this package's kernels are kept where they are within 2 % of the fastest (gemv before skinny)
            winners[M] = next((k for k in ("gemv", "skinny") if k in times and times[k] <= 1.02 * times[best]), best)
            cells = "  ".join(f"{k} {v:7.1f} us" for k, v in times.items())
            print(f"{name:8s} M={M:3d} N={N:6d} K={K:5d} ({N * K * 2 >> 20:4d} MiB)  {cells}  rule: {rule}"
                  + ("" if rule == best else f"  (fastest: {best}, {times[rule] / times[best]:.2f}x)"))
        print(f"    ({N}, {K}): {winners},")
        if name == "gate_up" or args.many_rows:
            gated = name == "gate_up"
            for M in (96, 128, 192, 256, 384, 512, 768, 1024, 1536, 2048, 3072, 4096, 8192):
                x = torch.randn(M, K, device="cuda", dtype=bf)
                if gated:
                    times = {"wide": time_calls(lambda i: gemm_bf16.wide(x, ws[i % len(ws)], bf, gated=True), args.iters, args.graph),
                             "pair": time_calls(lambda i: gemm_bf16.wide_pair(x, ws[i % len(ws)], bf, gated=True), args.iters, args.graph),
                             "product": time_calls(lambda i: ops.silu_mul(gemm_bf16._library(x, ws[i % len(ws)], bf)), args.iters, args.graph)}
                    rule = gemm_bf16.choose_gated(M, N, K)
                else:
                    times = {"pair": time_calls(lambda i: gemm_bf16.wide_pair(x, ws[i % len(ws)], out), args.iters, args.graph),
                             "library": time_calls(lambda i: gemm_bf16._library(x, ws[i % len(ws)], out), args.iters, args.graph)}
                    rule = gemm_bf16.choose(M, N, K)
                best = min(times, key=times.get)
                cells = "  ".join(f"{k} {v:8.1f} us" for k, v in times.items())
                print(f"{name:8s} M={M:4d}{' gated' if gated else ''}: {cells}  rule: {rule}"
                      + ("" if rule == best else f"  (fastest: {best}, {times[rule] / times[best]:.2f}x)"))
        del ws


def bench_step_timeline(args) -> None:
    """When every kernel of one decode step (a CUDA graph replay) starts and ends on the device, from
    the profiler's activity records: what lies on the critical path and what hides behind a neighbour."""
    from torch.profiler import ProfilerActivity, profile

    from tandem_b200.config.engine_config import EngineConfig
    from tandem_b200.engine.core import random_model
    from tandem_b200.engine.llm_engine import LLMEngine
    from tandem_b200.kernels import ops
    from tandem_b200.sampling.params import SamplingParams

    H = {"8b": 4096, "14b": 5120, "32b": 5120}[args.shapes]
    heads = {"8b": 32, "14b": 40, "32b": 64}[args.shapes]
    inter = {"8b": 12288, "14b": 17408, "32b": 25600}[args.shapes]
    config = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=args.layers, hidden_size=H,
                  num_attention_heads=heads, num_key_value_heads=8, head_dim=128, intermediate_size=inter, vocab_size=151936,
                  rope_theta=1e6, rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=args.context + 256)
    with torch.inference_mode(False):
        decoder, cfg = random_model(config, seed=0, dtype="bfloat16")
        pages = args.batch * (-(-(args.context + 64) // 16)) + 8
        eng = LLMEngine(EngineConfig(model="", dtype="bfloat16", block_size=16, num_kv_blocks=pages, max_num_seqs=args.batch,
                                     max_model_len=args.context + 256, cuda_graph_max_bs=args.batch),
                        decoder=decoder, model_config=cfg, load_tokenizer=False)
        g = torch.Generator().manual_seed(args.batch)
        sp = SamplingParams(max_tokens=64, temperature=0.0, ignore_eos=True)
        for _ in range(args.batch):
            eng.add_request(torch.randint(10, 100000, (args.context,), generator=g).tolist(), sp)
        while eng.scheduler.waiting or any(not r.is_decoding for r in eng.requests.values()):
            eng.step()
        for _ in range(8):
            eng.step()
        eng.drain()
        entries = eng.entries_of(eng.scheduler.schedule())
        for e in entries:
            e.want = [0]
        for _ in range(5):
            ops.argmax(eng.graphs.run(entries))
        torch.cuda.synchronize()
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            ops.argmax(eng.graphs.run(entries))
            torch.cuda.synchronize()
    events = sorted((e for e in prof.events() if e.device_time_total > 0 and "Memcpy" not in e.name), key=lambda e: e.time_range.start)
    t0 = events[0].time_range.start
    print(f"decode step, batch {args.batch}, context {args.context}, {args.layers} layers of Qwen3-{args.shapes} sizes: start, duration, end (us)")
    for e in events:
        start = e.time_range.start - t0
        print(f"{start:9.1f} +{e.device_time_total:7.1f} = {start + e.device_time_total:9.1f}  {e.name[:70]}")


def _cache(pages: int, nkv: int, ps: int, hd: int):
    return (torch.randn(pages, nkv, ps, hd, device="cuda", dtype=torch.bfloat16),
            torch.randn(pages, nkv, ps, hd, device="cuda", dtype=torch.bfloat16))


def bench_decode_attention(args) -> None:
    from tandem_b200.kernels import attention as A
    from tandem_b200.parts.base import KVView

    B, L, nh, nkv, hd, ps = args.batch, args.context, args.heads, args.kv_heads, args.head_dim, args.page_size
    pages_per_seq = -(-L // ps)
    kv_bytes = B * L * nkv * hd * 2 * 2
    copies = copies_for(kv_bytes)
    views = []
    for _ in range(copies):
        k, v = _cache(B * pages_per_seq, nkv, ps, hd)
        table = torch.randperm(B * pages_per_seq, device="cuda").to(torch.int32).view(B, pages_per_seq)
        views.append(KVView(k, v, table, None, ps, True))
    items = A.plan_decode([(b, b, L - 1) for b in range(B)], None, nkv, *([args.pieces * B * nkv] if args.pieces else []))
    spare = args.spare_items  # a CUDA graph's item array has room for the largest plan of its bucket: blocks without an item
    flat = torch.tensor([x for it in items for x in it] + [0] * (A.ITEM_INTS * spare), dtype=torch.int32, device="cuda")
    count = torch.tensor([len(items)], dtype=torch.int32, device="cuda")
    qkv = torch.randn(B, (nh + 2 * nkv) * hd, device="cuda", dtype=torch.bfloat16)
    us = time_calls(lambda i: A.paged_attention_decode(qkv, views[i % copies], flat, count, nh, nkv, hd, hd ** -0.5),
                    args.iters, args.graph)
    print(f"decode attention B={B} context={L} heads={nh}/{nkv} hd={hd} page={ps} items={len(items)}  {us:8.1f} us  "
          f"{kv_bytes / us / 1e3:7.0f} GB/s of keys and values")


def bench_prefill_attention(args) -> None:
    from tandem_b200.kernels import attention as A
    from tandem_b200.parts.base import KVView

    T, start, nh, nkv, hd, ps = args.tokens, args.start, args.heads, args.kv_heads, args.head_dim, args.page_size
    pages = -(-(start + T) // ps)
    k, v = _cache(pages, nkv, ps, hd)
    table = torch.randperm(pages, device="cuda").to(torch.int32).view(1, pages)
    kv = KVView(k, v, table, None, ps, True)
    flat = A.prefill_plan([(0, 0, start, T)], nh, nkv, hd, ps, None, "cuda")
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device="cuda", dtype=torch.bfloat16)
    us = time_calls(lambda i: A.paged_attention_prefill(qkv, kv, flat, nh, nkv, hd, None, hd ** -0.5), args.iters, args.graph)
    flops = 4.0 * nh * hd * (T * start + T * (T + 1) / 2)
    which = "tcgen05" if A.tcgen05_prefill_applies(hd, ps) else "mma.sync"
    print(f"prefill attention ({which}) tokens={T} start={start} heads={nh}/{nkv} hd={hd} page={ps} plan={tuple(flat.shape)}  {us:8.1f} us  "
          f"{flops / us / 1e6:7.1f} TFLOP/s")


def bench_tokenwise(args) -> None:
    from tandem_b200.kernels import ops

    T, H, I = args.tokens, args.hidden, args.intermediate
    bf = torch.bfloat16
    x, res, w = torch.randn(T, H, device="cuda", dtype=bf), torch.randn(T, H, device="cuda"), torch.ones(H, device="cuda")
    us = time_calls(lambda i: ops.add_rmsnorm(x, res, w, 1e-6, bf), args.iters, args.graph)
    print(f"add_rmsnorm T={T} H={H}  {us:8.1f} us  {T * H * 12 / us / 1e3:7.0f} GB/s")
    gu = torch.randn(T, 2 * I, device="cuda", dtype=bf)
    us = time_calls(lambda i: ops.silu_mul(gu), args.iters, args.graph)
    print(f"silu_mul    T={T} I={I}  {us:8.1f} us  {T * I * 6 / us / 1e3:7.0f} GB/s")
    nh, nkv, hd, ps = 32, 8, 128, 16
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device="cuda", dtype=bf)
    pages = -(-T // ps)
    kc, vc = _cache(pages, nkv, ps, hd)
    cs = torch.randn(max(T, 16), hd, device="cuda")
    pos = torch.arange(T, dtype=torch.int32, device="cuda")
    qw = torch.ones(hd, device="cuda")
    us = time_calls(lambda i: ops.qk_norm_rope_kv(qkv, pos, pos, qw, qw, cs, kc, vc, nh, nkv, hd, hd, ps, 1e-6), args.iters, args.graph)
    print(f"qk_norm_rope_kv T={T} heads={nh}/{nkv} hd={hd}  {us:8.1f} us  {T * (nh + 2 * nkv) * hd * 2 * 2 / us / 1e3:7.0f} GB/s")
    table = torch.randn(32768, H, device="cuda", dtype=bf)
    ids = torch.randint(0, 32768, (T,), device="cuda", dtype=torch.int32)
    us = time_calls(lambda i: ops.embedding(ids, table), args.iters, args.graph)
    print(f"embedding   T={T} H={H}  {us:8.1f} us  {T * H * 6 / us / 1e3:7.0f} GB/s")
    logits = torch.randn(min(T, 64), 151936, device="cuda")
    us = time_calls(lambda i: ops.argmax(logits), args.iters, args.graph)
    print(f"argmax      R={logits.shape[0]} V=151936  {us:8.1f} us  {logits.numel() * 4 / us / 1e3:7.0f} GB/s")


def bench_sampling(args) -> None:
    """From logits [rows, vocabulary] to tokens: argmax and the filters of temperature sampling, one by one
    and together, against one pass over the logits at memory speed."""
    from tandem_b200.kernels import ops

    R, V = args.rows, args.vocab
    logits = [torch.randn(R, V, device="cuda") * 3 for _ in range(copies_for(R * V * 4))]
    u = torch.rand(R, device="cuda")

    def opts(temperature=1.0, top_k=0, top_p=1.0, min_p=0.0):
        f = lambda v: torch.full((R,), v, device="cuda", dtype=torch.float32)
        return f(temperature), torch.full((R,), top_k, device="cuda", dtype=torch.int32), f(top_p), f(min_p)

    cases = [("argmax", None), ("temperature 0.8", opts(0.8)), ("top_k 50", opts(0.8, top_k=50)), ("top_p 0.9", opts(0.8, top_p=0.9)),
             ("min_p 0.05", opts(0.8, min_p=0.05)), ("top_k 50, top_p 0.9, min_p 0.05", opts(0.8, 50, 0.9, 0.05))]
    for name, o in cases:
        if o is None:
            us = time_calls(lambda i: ops.argmax(logits[i % len(logits)]), args.iters, args.graph)
        else:
            t, k, tp, mp = o
            any_k, any_p = bool(k[0] > 0), bool(tp[0] < 1)
            us = time_calls(lambda i: ops.sample(logits[i % len(logits)], t, k, tp, mp, u, any_top_k=any_k, any_top_p=any_p),
                            args.iters, args.graph)
        print(f"sampling R={R} V={V}  {name:32s} {us:8.1f} us  ({R * V * 4 / us / 1e3:6.0f} GB/s if it were one pass)")


def main(argv=None) -> None:
    p = argparse.ArgumentParser(prog="python -m tandem_b200.kernels.microbench")
    sub = p.add_subparsers(dest="case", required=True)
    common = argparse.ArgumentParser(add_help=False)
    common.add_argument("--iters", type=int, default=20)
    common.add_argument("--no-graph", dest="graph", action="store_false")
    g = sub.add_parser("gemm", parents=[common])
    g.add_argument("--m", type=int, default=8)
    g.add_argument("--n", type=int, default=24576)
    g.add_argument("--k", type=int, default=4096)
    g.add_argument("--f32-out", action="store_true")
    g.add_argument("--gated", action="store_true", help="also time the product with the SiLU * up epilogue (rows of W = [gate | up])")
    g.add_argument("--impl", choices=["both", "skinny", "gemv", "wide", "pair", "library"], default="both")
    g.set_defaults(fn=bench_gemm)
    ng = sub.add_parser("norm-gemm", parents=[common])
    ng.add_argument("--m", type=int, default=8)
    ng.add_argument("--n", type=int, default=6144)
    ng.add_argument("--k", type=int, default=4096)
    ng.set_defaults(fn=bench_norm_gemm)
    shape = argparse.ArgumentParser(add_help=False)
    shape.add_argument("--heads", type=int, default=32)
    shape.add_argument("--kv-heads", type=int, default=8)
    shape.add_argument("--head-dim", type=int, default=128)
    shape.add_argument("--page-size", type=int, default=16)
    d = sub.add_parser("decode-attention", parents=[common, shape])
    d.add_argument("--batch", type=int, default=64)
    d.add_argument("--context", type=int, default=2048)
    d.add_argument("--pieces", type=int, default=0, help="cut every request's keys into this many items instead of what the rule picks")
    d.add_argument("--spare-items", type=int, default=0, help="room in the item array beyond the plan, as in a CUDA graph's bucket")
    d.set_defaults(fn=bench_decode_attention)
    f = sub.add_parser("prefill-attention", parents=[common, shape])
    f.add_argument("--tokens", type=int, default=2048)
    f.add_argument("--start", type=int, default=0)
    f.set_defaults(fn=bench_prefill_attention)
    t = sub.add_parser("tokenwise", parents=[common])
    t.add_argument("--tokens", type=int, default=2048)
    t.add_argument("--hidden", type=int, default=4096)
    t.add_argument("--intermediate", type=int, default=12288)
    t.set_defaults(fn=bench_tokenwise)
    sa = sub.add_parser("sampling", parents=[common])
    sa.add_argument("--rows", type=int, default=64)
    sa.add_argument("--vocab", type=int, default=151936)
    sa.set_defaults(fn=bench_sampling)
    dp = sub.add_parser("dispatch", parents=[common])
    dp.add_argument("--shapes", choices=sorted(LAYER_SHAPES), default="8b")
    dp.add_argument("--many-rows", action="store_true", help="also the pair kernel against the library at 96 to 8,192 rows, every product")
    dp.set_defaults(fn=bench_dispatch)
    tl = sub.add_parser("step-timeline", parents=[common])
    tl.add_argument("--batch", type=int, default=8)
    tl.add_argument("--context", type=int, default=2048)
    tl.add_argument("--layers", type=int, default=4)
    tl.add_argument("--shapes", choices=sorted(LAYER_SHAPES), default="8b")
    tl.set_defaults(fn=bench_step_timeline)
    args = p.parse_args(argv)
    with torch.inference_mode():
        args.fn(args)


if __name__ == "__main__":
    main()
