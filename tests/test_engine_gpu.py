"""The engine on the GPU: generation through the entry point, long decoding, the first tokens of a
sequence, preemption, temperature sampling, each part alone, and parts defined outside the package."""

import subprocess
import sys
from dataclasses import dataclass, replace

import pytest
import torch

import plain_qwen3 as plain
from conftest import ROOT, TINY, random_tokens

pytestmark = pytest.mark.gpu

GREEDY = dict(temperature=0.0, ignore_eos=True)


def near_tie(cfg, w, prompt, got, want, gap=0.05):
    """bfloat16 greedy may leave the float32 path only where the plain logits nearly tie
    (tests/test_gpu_fastpath.py:81-92 of 12vivi/tandem)."""
    for i, (x, y) in enumerate(zip(got, want)):
        if x != y:
            logits = plain.forward(cfg, w, prompt + want[:i])[-1]
            return abs(float(logits[x] - logits[y])) < gap
    return True


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,lengths,budget,policy,new", [("A", [5, 17, 33], 16, "prefill_first", 8),
                                                            ("B", [1, 9, 40, 70], 16, "decode_first", 12),
                                                            ("C", [30, 3, 61], 24, "decode_first", 40)])
def test_greedy_generation_through_the_entry_point(tiny_folder, name, lengths, budget, policy, new, dtype):
    from tandem_b200 import LLM, SamplingParams

    folder = tiny_folder(name, 0.1)
    cfg, w = plain.read_folder(folder)
    prompts = [random_tokens(7 + i, n, TINY[name]["vocab_size"]) for i, n in enumerate(lengths)]
    llm = LLM(model=folder, dtype=dtype, block_size=8, num_kv_blocks=64, max_num_batched_tokens=budget,
              schedule_policy=policy, max_num_seqs=4)
    outs = llm.generate(prompts, SamplingParams(max_tokens=new, **GREEDY))
    for p, o in zip(prompts, outs):
        want = plain.greedy(cfg, w, p, new)
        assert o.finish_reason == "length" and len(o.output_token_ids) == new
        if dtype == "float32":
            assert o.output_token_ids == want
        else:
            assert near_tie(cfg, w, p, o.output_token_ids, want)
    assert llm.engine.cache.all_free()  # every page and slot given back
    assert llm.stats()["free_kv_blocks"] == llm.stats()["total_kv_blocks"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_recomputes_exactly(tiny_folder, dtype):
    """12 pages of 4 tokens cannot hold four requests of 10 + 14 tokens: some are preempted and
    recomputed, and the outputs stay those of the plain implementation
    (tests/test_model_equivalence.py:55-64 of 12vivi/tandem)."""
    from tandem_b200 import EngineConfig, LLMEngine, SamplingParams

    folder = tiny_folder("A", 0.1)
    cfg, w = plain.read_folder(folder)
    eng = LLMEngine(EngineConfig(model=folder, dtype=dtype, block_size=4, num_kv_blocks=12, max_num_batched_tokens=16,
                                 schedule_policy="decode_first"))
    prompts = [random_tokens(40 + i, 10, 512) for i in range(4)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=14, **GREEDY))
    assert eng.scheduler.num_preemptions > 0
    for p, o in zip(prompts, outs):
        want = plain.greedy(cfg, w, p, 14)
        assert o.output_token_ids == want if dtype == "float32" else near_tie(cfg, w, p, o.output_token_ids, want)
    eng.cache.check()
    assert eng.cache.all_free()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(tiny_folder, dtype):
    """One token at a time from position 0 to 300 (the first tokens of a sequence: a single key,
    a page's first slot) and on through many pages; logits against the plain implementation."""
    from tandem_b200.engine.core import build_executor, load_model
    from tandem_b200.engine.executor import StepEntry

    folder = tiny_folder("B")
    cfg, w = plain.read_folder(folder, torch.float64)
    tokens = random_tokens(3, 300, 1000)
    ref = plain.forward(cfg, w, tokens, torch.float64)
    decoder, _ = load_model(folder, dtype, "cuda:0")
    ex = build_executor(decoder, page_size=16, num_pages=20, max_requests=2)
    rows = [ex.step([StepEntry("a", [t], [0])]) for t in tokens]
    got = torch.cat(rows).cpu().double()
    err = (got - ref).abs().max(-1).values
    assert err[:4].max() < (1e-4 if dtype == "float32" else 0.05)
    assert err.max() < (1e-4 if dtype == "float32" else 0.08), int(err.argmax())


def test_cuda_graph_decode_matches_eager(tiny_folder):
    """Decode-only steps replayed from CUDA graphs (batches padded up to a bucket, static batch
    description) give the logits of the eager step function, step after step, as requests come and go."""
    from tandem_b200.engine.core import build_executor, load_model
    from tandem_b200.engine.cuda_graph import DecodeGraphs, bucket_sizes
    from tandem_b200.engine.executor import StepEntry

    assert bucket_sizes(64) == [1, 2, 4, 8, 12, 16, 24, 32, 40, 48, 56, 64] and bucket_sizes(5) == [1, 2, 4, 5]
    decoder, _ = load_model(tiny_folder("B"), "bfloat16", "cuda:0")
    eager = build_executor(decoder, page_size=16, num_pages=64, max_requests=8)
    graph = build_executor(decoder, page_size=16, num_pages=64, max_requests=8)
    graphs = DecodeGraphs.maybe(graph, 8, 512)
    assert graphs is not None
    prompts = {f"r{i}": random_tokens(80 + i, n, 1000) for i, n in enumerate([3, 70, 129, 17, 40])}
    for ex in (eager, graph):
        ex.step([StepEntry(rid, t, []) for rid, t in prompts.items()])
    live = list(prompts)
    for step in range(40):
        if step in (7, 19, 30):  # a request ends: the batch shrinks, another bucket takes over
            gone = live.pop(0)
            eager.manager.end(gone), graph.manager.end(gone)
        entries = [StepEntry(rid, [(step * 7 + i) % 1000], [0]) for i, rid in enumerate(live)]
        assert graphs.takes(entries)
        for ex in (eager, graph):
            for e in entries:
                assert ex.manager.grow(e.request_id, ex.manager.num_tokens(e.request_id) + 1)
        a = eager.run(entries)
        b = graphs.run(entries).clone()
        for ex in (eager, graph):
            for e in entries:
                ex.manager.commit(e.request_id, 1)
        assert (a - b).abs().max() < 0.06, step  # bfloat16 rounding only (the padded batch may pick other GEMM tiles)
    assert len(graphs.captured) >= 3 and all(c.launches > 0 for c in graphs.captured.values())
    assert not graphs.takes([StepEntry(live[0], [1, 2], [1])])


@pytest.mark.parametrize("name,page", [("B", 16), ("A", 16), ("C", 16)])
def test_cuda_graph_decode_follows_the_plain_implementation(tiny_folder, name, page):
    """Decode steps replayed from CUDA graphs against the plain logits: three live requests (the
    bucket of 4, one padding row), then five (the bucket of 8, three padding rows), then three
    others (the bucket of 4 again, replayed with other requests on pages that finished requests
    gave back), then two.  Every request is fed its own given tokens, so each row of logits has a
    place in the plain implementation's whole-sequence output."""
    import replay_cases as rc
    from tandem_b200.engine.core import build_executor, load_model
    from tandem_b200.engine.cuda_graph import DecodeGraphs
    from tandem_b200.engine.executor import StepEntry

    folder = tiny_folder(name)
    vocab = TINY[name]["vocab_size"]
    cfg, w64 = plain.read_folder(folder, torch.float64)
    _, w16 = plain.read_folder(folder, torch.bfloat16)
    lengths = {"r0": 70, "r1": 45, "r2": 100, "r3": 33, "r4": 120, "r5": 90}
    head = {"r0": 50, "r1": 30, "r2": 81, "r3": 2, "r4": 97, "r5": 64}  # tokens read as one portion; the rest one by one
    toks = {rid: random_tokens(500 + i, n, vocab) for i, (rid, n) in enumerate(lengths.items())}
    decoder, _ = load_model(folder, "bfloat16", "cuda:0")
    ex = build_executor(decoder, page_size=page, num_pages=23, max_requests=8)
    log = rc.PageLog(ex.manager)
    graphs = DecodeGraphs.maybe(ex, 8, 256)
    assert graphs is not None
    at, got = {}, {rid: {} for rid in toks}

    def admit(*rids):
        ex.step([StepEntry(rid, toks[rid][: head[rid]], []) for rid in rids])
        for rid in rids:
            at[rid] = head[rid]

    def decode(live, steps):
        for _ in range(steps):
            entries = [StepEntry(rid, [toks[rid][at[rid]]], [0]) for rid in live if at[rid] < lengths[rid]]
            assert graphs.takes(entries)
            for e in entries:
                assert ex.manager.grow(e.request_id, at[e.request_id] + 1)
            logits = graphs.run(entries).double().cpu()
            for row, e in zip(logits, entries):
                ex.manager.commit(e.request_id, 1)
                got[e.request_id][at[e.request_id]] = row
                at[e.request_id] += 1
            ex.manager.check()

    admit("r0", "r1", "r2")
    decode(["r0", "r1", "r2"], 9)  # eager + capture of bucket 4, then replays
    admit("r3", "r4")
    decode(["r0", "r1", "r2", "r3", "r4"], 6)  # bucket 8
    for rid in ("r0", "r1", "r2"):
        ex.manager.end(rid)
    admit("r5")  # onto pages that r0..r2 held
    decode(["r3", "r4", "r5"], 12)  # bucket 4 replayed with other requests and other pages
    ex.manager.end("r3")
    decode(["r4", "r5"], 11)  # bucket 2
    ex.manager.end("r4"), ex.manager.end("r5")
    assert ex.manager.all_free()
    assert set(graphs.captured) >= {2, 4, 8} and log.reused_beside_live >= 3
    for rid, rows in got.items():
        assert rows, rid
        ref = plain.forward(cfg, w64, toks[rid], torch.float64)
        low = plain.forward(cfg, w16, toks[rid], torch.bfloat16).double()
        base = (low - ref).abs().max().item()
        for pos, row in rows.items():
            err = (row - ref[pos]).abs().max().item()
            assert err <= 1.5 * base + 0.02, (rid, pos, err, base)


def test_cuda_graphs_take_short_steps_with_prompt_portions(tmp_path):
    """Steps of up to 256 tokens that bring prompt portions are replayed from CUDA graphs too (where the
    tcgen05 prefill kernel applies: a head size of 64 here): portions of 2 to 40 tokens of up to four
    requests beside single tokens of others, padded to buckets of 16 to 128 token rows, on pages that
    finished requests gave back; every row of logits against the plain implementation."""
    import replay_cases as rc
    from tandem_b200.engine.core import build_executor, load_model
    from tandem_b200.engine.cuda_graph import DecodeGraphs
    from tandem_b200.engine.executor import StepEntry
    from tandem_b200.weights.random_init import write_random_model

    config = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=136,
                  num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=264, vocab_size=1003,
                  rope_theta=50000.0, rms_norm_eps=2e-6, tie_word_embeddings=False, max_position_embeddings=512)
    folder = str(tmp_path / "hd64")
    write_random_model(config, folder, seed=11, dtype="bfloat16", std=0.05)
    cfg, w64 = plain.read_folder(folder, torch.float64)
    _, w16 = plain.read_folder(folder, torch.bfloat16)
    g = torch.Generator().manual_seed(77)
    lengths = {f"r{i}": int(n) for i, n in enumerate(torch.randint(40, 200, (9,), generator=g))}
    toks = {rid: random_tokens(900 + i, n, 1003) for i, (rid, n) in enumerate(lengths.items())}
    decoder, _ = load_model(folder, "bfloat16", "cuda:0")
    ex = build_executor(decoder, page_size=16, num_pages=40, max_requests=8)
    log = rc.PageLog(ex.manager)
    graphs = DecodeGraphs.maybe(ex, 8, 512)
    assert graphs is not None and graphs.mixed
    at = {rid: 0 for rid in toks}
    got = {rid: {} for rid in toks}
    waiting, live, steps, replayed_before = list(toks), [], 0, 0
    while waiting or live:
        while waiting and len(live) < 4 and ex.manager.free_pages(0) * 16 >= lengths[waiting[0]] + 16:
            rid = waiting.pop(0)
            ex.manager.begin(rid)
            live.append(rid)
        entries = []
        for rid in live:
            left = lengths[rid] - at[rid]
            # most steps cut prompts into short portions; a request near its end goes token by token
            n = 1 if left <= 12 else min(left, int(torch.randint(2, 41, (1,), generator=g)))
            entries.append(StepEntry(rid, toks[rid][at[rid]: at[rid] + n], [n - 1] if n > 1 or left <= 12 else []))
        for e in entries:
            assert ex.manager.grow(e.request_id, at[e.request_id] + len(e.tokens))
        if graphs.takes(entries):
            logits = graphs.run(entries).double().cpu()
        else:
            assert sum(len(e.tokens) for e in entries) > 256 or sum(len(e.want) for e in entries) > 8
            logits = ex.run(entries).double().cpu()
        row = 0
        for e in entries:
            ex.manager.commit(e.request_id, len(e.tokens))
            for w in e.want:
                got[e.request_id][at[e.request_id] + w] = logits[row]
                row += 1
            at[e.request_id] += len(e.tokens)
        assert row == logits.shape[0]
        for rid in [r for r in live if at[r] >= lengths[r]]:
            ex.manager.end(rid)
            live.remove(rid)
        ex.manager.check()
        steps += 1
    assert ex.manager.all_free() and log.reused_beside_live >= 2
    mixed = {k: c for k, c in graphs.captured.items() if isinstance(k, tuple)}
    assert len(mixed) >= 3 and sum(c.replays for c in mixed.values()) >= 10, {k: c.replays for k, c in graphs.captured.items()}
    assert graphs.mixed_fallbacks == 0
    for rid, rows in got.items():
        assert rows, rid
        ref = plain.forward(cfg, w64, toks[rid], torch.float64)
        low = plain.forward(cfg, w16, toks[rid], torch.bfloat16).double()
        base = (low - ref).abs().max().item()
        for pos, row in rows.items():
            err = (row - ref[pos]).abs().max().item()
            assert err <= 1.5 * base + 0.02, (rid, pos, err, base)
    from tandem_b200.kernels import ops as kernel_ops

    kernel_ops.check_status("cuda")


def test_a_fault_recorded_by_a_kernel_stops_the_engine(tiny_folder):
    """Kernels that survive a fault (a bounded wait that gave up, a missing page) record it in a
    status word; the engine reads the word with the step's tokens and raises instead of handing
    out tokens sampled from invalid logits.  The word is set by hand here."""
    from tandem_b200 import EngineConfig, LLMEngine, SamplingParams
    from tandem_b200.kernels import ops

    for overlap in (False, True):
        eng = LLMEngine(EngineConfig(model=tiny_folder("A"), dtype="bfloat16", block_size=16, num_kv_blocks=16,
                                     overlap_schedule=overlap))
        eng.add_request([5, 6, 7], SamplingParams(max_tokens=8, **GREEDY))
        eng.step()
        with torch.inference_mode():
            ops.status_word(eng.decoder.device).fill_(2)
        with pytest.raises(ops.KernelError, match="missing page"):
            for _ in range(3):
                eng.step()
        assert int(ops.status_word(eng.decoder.device).item()) == 0  # cleared: the next engine starts clean


def test_replayed_graphs_keep_the_scratch_they_were_captured_with(tiny_folder):
    """The decode kernel's scratch grows with the batch; a graph captured before it grew still
    writes to the scratch of its day when it is replayed, so that memory must not go to anyone else."""
    from tandem_b200.engine.core import build_executor, load_model
    from tandem_b200.engine.cuda_graph import DecodeGraphs
    from tandem_b200.engine.executor import StepEntry
    from tandem_b200.kernels import attention as attention_kernels

    decoder, cfg = load_model(tiny_folder("B"), "bfloat16", "cuda:0")
    ex = build_executor(decoder, page_size=16, num_pages=64, max_requests=8)
    graphs = DecodeGraphs.maybe(ex, 8, 512)
    ex.step([StepEntry("a", random_tokens(5, 450, 1000), [])])  # long enough to be cut into two items

    def decode(token):
        assert ex.manager.grow("a", ex.manager.num_tokens("a") + 1)
        logits = graphs.run([StepEntry("a", [token], [0])]).clone()
        ex.manager.commit("a", 1)
        return logits

    decode(1), decode(2)  # eager and capture, then a replay
    ws = attention_kernels._workspaces["cuda:0"]
    sizes = [ws["part_o"].numel(), ws["part_ml"].numel()]
    heads = cfg.num_attention_heads
    grown = attention_kernels._workspace(decoder.device, 2 * ws["rows"] // heads + 1, cfg.num_key_value_heads,
                                         heads // cfg.num_key_value_heads, cfg.head_dim)
    assert grown is not ws
    del ws
    canaries = [torch.zeros(n, dtype=torch.float32, device=decoder.device) for n in sizes for _ in range(4)]
    decode(3)  # the graph of bucket 1, captured with the scratch that has been outgrown
    torch.cuda.synchronize()
    assert all(int(c.count_nonzero()) == 0 for c in canaries)


def test_generation_with_cuda_graphs(tiny_folder):
    from tandem_b200 import LLM, SamplingParams

    folder = tiny_folder("A", 0.1)
    cfg, w = plain.read_folder(folder)
    prompts = [random_tokens(90 + i, n, 512) for i, n in enumerate([4, 30, 11])]
    llm = LLM(model=folder, dtype="bfloat16", block_size=16, num_kv_blocks=32, max_num_seqs=4, cuda_graph=True)
    assert llm.engine.graphs is not None
    outs = llm.generate(prompts, SamplingParams(max_tokens=20, **GREEDY))
    assert llm.engine.graphs.captured
    for p, o in zip(prompts, outs):
        assert near_tie(cfg, w, p, o.output_token_ids, plain.greedy(cfg, w, p, 20))
    assert llm.engine.cache.all_free()


def test_qwen3_8b_widths_follow_the_plain_implementation_however_they_are_cut():
    """The real layer sizes (hidden 4096, 32 query and 8 kv heads of 128, intermediate 12288,
    vocabulary 151936, pages of 16), three layers of them with random weights made on the device:
    a 330-token request whole, in portions with its last 30 tokens one by one, and beside another
    request whose pages it later reuses.  The float32 path gives the same bits however it is cut,
    and those bits are the plain implementation's float64 logits to float32 rounding; bfloat16
    stays within what its 8-bit mantissa allows (about 1 % of the logits' spread on average; the
    bounds below leave a factor of two)."""
    from bench import QWEN3_8B
    from tandem_b200.engine.core import build_executor, random_model
    from tandem_b200.engine.executor import StepEntry
    from tandem_b200.registry import resolve_architecture

    tokens, other = random_tokens(1, 330, 151936), random_tokens(2, 200, 151936)
    results = {}
    for dtype in ("float32", "bfloat16"):
        decoder, _ = random_model(QWEN3_8B, seed=3, dtype=dtype, num_layers=3, stored_dtype="bfloat16")
        ex = build_executor(decoder, page_size=16, num_pages=30, max_requests=4)
        whole = ex.step([StepEntry("w", tokens, list(range(300, 330)))], end=["w"])
        cut, at = [], 0
        for n in [130, 2, 61, 9, 12, 14, 72] + [1] * 30:  # 9 to 14 rows: the streaming products' two-tile form, add and norm riding along
            out = ex.step([StepEntry("p", tokens[at: at + n], [i for i in range(n) if at + i >= 300])])
            at += n
            cut.append(out)
        ex.step([], end=["p"])
        # beside another request, in a pool of 30 pages that the two fill but for one: the end of the
        # long request lands on pages the other one has given back
        mixed = [ex.step([StepEntry("o", other, []), StepEntry("m", tokens[:200], [])])]
        mixed.append(ex.step([StepEntry("o", [5], [0]), StepEntry("m", tokens[200:250], [])], end=["o"]))
        assert ex.manager.free_pages(0) == 14
        mixed = [ex.step([StepEntry("m", tokens[250:], list(range(50, 80)))], end=["m"])]
        assert ex.manager.all_free()
        results[dtype] = [whole.double().cpu(), torch.cat([c for c in cut if c.shape[0]]).double().cpu(), mixed[0].double().cpu()]
        del decoder, ex
        torch.cuda.empty_cache()
    f32, b16 = results["float32"], results["bfloat16"]
    assert torch.equal(f32[0], f32[1]) and torch.equal(f32[0], f32[2])
    spread = f32[0].std().item()
    assert spread > 0.5  # the logits are not degenerate
    # the same tensors (same seeds, drawn on the same device) through the plain implementation in float64
    arch = resolve_architecture(QWEN3_8B)
    cfg3 = dict(QWEN3_8B, num_hidden_layers=3)
    weights = {n: t.cpu().double() for n, t in arch.random_weights(arch.config_class.from_dict(cfg3), 3, "cuda:0", torch.bfloat16)}
    ref = plain.forward(cfg3, weights, tokens, torch.float64)[300:]
    del weights
    err = (f32[0] - ref).abs().max().item()
    assert err < 1e-4 * max(1.0, ref.abs().max().item()), (err, ref.abs().max().item(), spread)
    for got in b16:
        err = (got - f32[0]).abs()
        assert err.mean().item() < 0.025 * spread and err.max().item() < 0.15 * spread, (err.mean().item(), err.max().item(), spread)


def test_temperature_sampling_is_seeded_and_independent_of_the_batch(tiny_folder):
    from tandem_b200 import EngineConfig, LLMEngine, SamplingParams

    folder = tiny_folder("B", 0.1)
    prompts = [random_tokens(60 + i, n, 1000) for i, n in enumerate([1, 9, 40, 70])]
    sp = [SamplingParams(max_tokens=12, temperature=0.8, top_p=0.9, seed=42 + i, ignore_eos=True) for i in range(4)]

    def run(which, budget, policy):
        eng = LLMEngine(EngineConfig(model=folder, dtype="float32", block_size=8, num_kv_blocks=64,
                                     max_num_batched_tokens=budget, schedule_policy=policy))
        return [o.output_token_ids for o in eng.generate([prompts[i] for i in which], [sp[i] for i in which])]

    together = run([0, 1, 2, 3], 16, "decode_first")
    assert together == run([0, 1, 2, 3], 16, "decode_first")  # reproducible (tests/test_spec_and_sampling.py:82-88)
    alone = [run([i], 64, "prefill_first")[0] for i in range(4)]
    assert together == alone  # a draw depends on (seed, index of the token) only
    assert len({tuple(t) for t in together}) == 4
    # and the draws follow the plain sampler on the plain logits
    cfg, w = plain.read_folder(folder)
    from tandem_b200.sampling.rng import uniform

    ids = list(prompts[1])
    for k, tok in enumerate(alone[1][:4]):
        p = plain.filtered_probs(plain.forward(cfg, w, ids)[-1], 0.8, top_p=0.9)
        want = plain.inverse_cdf_draw(p, uniform(43, k))
        assert tok == want
        ids.append(tok)


def test_temperature_sampling_in_bfloat16_is_reproducible(tiny_folder):
    """Which kernel computes a product is fixed, so a bfloat16 run gives the same logits, and with
    seeded draws the same tokens, every time; with other seeds it gives other tokens."""
    from tandem_b200 import EngineConfig, LLMEngine, SamplingParams

    folder = tiny_folder("B", 0.1)
    prompts = [random_tokens(160 + i, n, 1000) for i, n in enumerate([3, 20, 45])]

    def run(seed):
        sp = [SamplingParams(max_tokens=16, temperature=0.9, top_k=40, top_p=0.95, min_p=0.01, seed=seed + i, ignore_eos=True)
              for i in range(3)]
        eng = LLMEngine(EngineConfig(model=folder, dtype="bfloat16", block_size=16, num_kv_blocks=32, max_num_batched_tokens=32))
        outs = eng.generate(prompts, sp)
        assert eng.cache.all_free() and all(0 <= t < 1000 for o in outs for t in o.output_token_ids)
        return [o.output_token_ids for o in outs]

    first = run(7)
    assert first == run(7)
    assert first != run(8)


class LetterTokenizer:
    """One letter per token id."""

    def encode(self, text):
        return [ord(c) - 97 for c in text]

    def decode(self, ids, skip_special_tokens=True):
        return "".join(chr(97 + i % 26) for i in ids)


@pytest.mark.parametrize("overlap", [False, True])
def test_stop_strings_end_a_request_and_need_a_tokenizer(tiny_folder, overlap):
    from tandem_b200 import EngineConfig, LLMEngine, SamplingParams

    folder = tiny_folder("A", 0.1)
    cfg, w = plain.read_folder(folder)
    tok = LetterTokenizer()
    prompts = [random_tokens(70 + i, n, 512) for i, n in enumerate([6, 19])]
    want = [plain.greedy(cfg, w, p, 16) for p in prompts]
    texts = [tok.decode(t) for t in want]
    stop = texts[0][7:10]  # the first request stops where these three letters first appear; the second runs on
    ends = [t.find(stop) for t in texts]
    config = EngineConfig(model=folder, dtype="float32", block_size=8, num_kv_blocks=32, overlap_schedule=overlap)
    eng = LLMEngine(config, tokenizer=tok)
    outs = eng.generate(prompts, [SamplingParams(max_tokens=16, stop=[stop], **GREEDY), SamplingParams(max_tokens=16, **GREEDY)])
    assert outs[0].finish_reason == "stop" and outs[0].text == texts[0][: ends[0]]
    assert outs[0].output_token_ids == want[0][: ends[0] + 3]  # tokens up to the one that completed the stop string
    assert outs[1].finish_reason == "length" and outs[1].text == texts[1] and outs[1].output_token_ids == want[1]
    assert eng.cache.all_free()
    with pytest.raises(ValueError, match="tokenizer"):
        LLMEngine(config, load_tokenizer=False).add_request(prompts[0], SamplingParams(stop=["x"]))


def test_command_line(tiny_folder):
    out = subprocess.run([sys.executable, f"{ROOT}/bin/tandem", "generate", "--model", tiny_folder("A", 0.1), "--dtype", "float32",
                          "--prompt-ids", "5 17 3 99", "--max-tokens", "5", "--temperature", "0", "--ignore-eos",
                          "--block-size", "4", "--kv-cache-gb", "0.001"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    cfg, w = plain.read_folder(tiny_folder("A", 0.1))
    assert [int(t) for t in out.stdout.split()] == plain.greedy(cfg, w, [5, 17, 3, 99], 5)
    assert "tok/s" in out.stderr and "free_kv_blocks" in out.stderr


# ----------------------------------------------------------------------------- parts alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_each_part_alone(dtype):
    """Norm, feed-forward, position table and attention mixer built from specs with sizes of
    their own (no model around them) against the plain functions."""
    from tandem_b200.cache.manager import CacheManager
    from tandem_b200.cache.storage import CacheStorage
    from tandem_b200.config.plan import AttentionSpec, GatedMLPSpec, NormSpec, PositionSpec
    from tandem_b200.engine.executor import Executor, StepEntry
    from tandem_b200.parts.attention import PagedAttention
    from tandem_b200.parts.mlp import GatedMLP
    from tandem_b200.parts.norm import RMSNorm
    from tandem_b200.parts.rope import RotaryTable

    g = torch.Generator().manual_seed(0)
    tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=3e-2, rtol=3e-2)
    H, I, nh, nkv, hd, T = 72, 100, 6, 3, 48, 21

    def rnd(*shape, s=1.0):
        return (torch.randn(*shape, generator=g) * s).to(dtype)

    # norm
    wn = 1 + 0.1 * torch.randn(H, generator=g)
    norm = RMSNorm(NormSpec("rmsnorm", H, 1e-5, "n"), {"weight": wn.cuda()}, dtype, "cuda")
    x, res = rnd(T, H), torch.randn(T, H, generator=g)
    y = norm.forward(x.cuda(), res.clone().cuda(), dtype)
    torch.testing.assert_close(y.cpu().float(), plain.rms_norm(x.float() + res, wn, 1e-5), **tol)

    # feed-forward
    wg, wu, wd = rnd(I, H, s=0.2), rnd(I, H, s=0.2), rnd(H, I, s=0.2)
    mlp = GatedMLP(GatedMLPSpec("gated_mlp", "m", H, I), {"gate_up": torch.cat([wg, wu]).cuda(), "down": wd.cuda()}, dtype, "cuda")
    wdict = {"m.gate_proj.weight": wg.float(), "m.up_proj.weight": wu.float(), "m.down_proj.weight": wd.float()}
    torch.testing.assert_close(mlp.forward(x.cuda(), None).cpu().float(), plain.swiglu(x.float(), wdict, "m"), **tol)

    # position table
    table = RotaryTable(PositionSpec("rope", rotary_dim=hd, theta=777.0, max_position=64), "cuda")
    cos, sin = plain.rope_tables(hd, 777.0, 64, torch.float32)
    torch.testing.assert_close(table.cos_sin.cpu(), torch.cat([cos[:, : hd // 2], sin[:, : hd // 2]], 1), atol=0, rtol=0)

    # attention mixer, two portions of one request through a cache of its own
    spec = AttentionSpec("attention", prefix="a", hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                         scale=hd ** -0.5, qk_norm=True, qk_norm_eps=1e-5, window=None,
                         position=PositionSpec("rope", rotary_dim=hd, theta=777.0, max_position=64))
    wq, wk, wv, wo = rnd(nh * hd, H, s=0.2), rnd(nkv * hd, H, s=0.2), rnd(nkv * hd, H, s=0.2), rnd(H, nh * hd, s=0.2)
    qn, kn = 1 + 0.1 * torch.randn(hd, generator=g), 1 + 0.1 * torch.randn(hd, generator=g)
    mixer = PagedAttention(spec, {"qkv": torch.cat([wq, wk, wv]).cuda(), "o": wo.cuda(), "q_norm": qn.cuda(), "k_norm": kn.cuda()},
                           dtype, "cuda")
    need = PagedAttention.kv_need(spec)
    manager = CacheManager([need], page_size=8, num_pages=4, max_requests=2)
    storage = CacheStorage(manager, [need], [None], [None], dtype, "cuda")

    class OneMixer:  # the smallest thing the executor's batch builder needs around a mixer
        dtype, device = mixer.qkv.dtype, torch.device("cuda")

        class plan:
            max_position = 64

            class embedding:
                vocab_size = 10

    ex = Executor(OneMixer, manager, storage)
    outs = []
    for start, n in ((0, 13), (13, 8)):
        manager.begin("r") if start == 0 else None
        assert manager.grow("r", start + n)
        ctx, _ = ex.build_context([StepEntry("r", [0] * n, [])])
        ctx.run = 0
        outs.append(mixer.forward(x[start: start + n].cuda(), ctx))
        manager.commit("r", n)
    d = dict(nh=nh, nkv=nkv, hd=hd, eps=1e-5)
    wdict = {"a.q_proj.weight": wq.float(), "a.k_proj.weight": wk.float(), "a.v_proj.weight": wv.float(),
             "a.o_proj.weight": wo.float(), "a.q_norm.weight": qn, "a.k_norm.weight": kn}
    cos, sin = plain.rope_tables(hd, 777.0, T, torch.float32)
    want = plain.attention_block(x.float(), wdict, "a", d, cos, sin, None)
    torch.testing.assert_close(torch.cat(outs).cpu().float(), want, atol=tol["atol"] * 4, rtol=tol["rtol"])


# ----------------------------------------------------------------------------- parts from outside
@dataclass(frozen=True)
class DecaySpec:
    """A toy mixer with state of its own: y_t = x_t + s_t, s_t = decay * s_{t-1} + x_t @ W,
    s kept per request in a state slot of fixed size (hidden floats)."""

    family = "mixer"  # which kind of part this is a spec of (the package's own specs inherit it from MixerSpec)
    kind: str = "toy_decay"
    prefix: str = ""
    hidden_size: int = 0
    decay: float = 0.5


class DecayMixer:
    @staticmethod
    def params(spec):
        from tandem_b200.config.plan import ParamSpec, WeightSource

        return {"w": ParamSpec((spec.hidden_size, spec.hidden_size), (WeightSource(f"{spec.prefix}.w"),))}

    @staticmethod
    def kv_need(spec):
        return None

    @staticmethod
    def state_need(spec):
        from tandem_b200.parts.base import StateNeed

        return StateNeed((spec.hidden_size,), torch.float32)

    def __init__(self, spec, weights, dtype, device):
        self.spec, self.w = spec, weights["w"]

    def forward(self, x, ctx):
        state = ctx.state()
        u = (x.float() @ self.w.float().T)
        out = torch.empty_like(u)
        at = 0
        for slot, n in zip(ctx.host_slots, ctx.host_lens):  # the step's requests, in order
            s = state[slot]
            for t in range(at, at + n):
                s = self.spec.decay * s + u[t]
                out[t] = x[t].float() + s
            state[slot] = s
            at += n
        return out.to(x.dtype)


def _toy_plan(vocab, H, layers):
    from tandem_b200.config.plan import EmbeddingSpec, GatedMLPSpec, HeadSpec, LayerSpec, ModelPlan, NormSpec, RunStep

    return ModelPlan(
        embedding=EmbeddingSpec(vocab, H, "emb"),
        layers=tuple(LayerSpec.of("prenorm", mixer=m, feed_forward=GatedMLPSpec("gated_mlp", f"l{i}.mlp", H, 2 * H),
                               mixer_norm=NormSpec("rmsnorm", H, 1e-5, f"l{i}.n1"),
                               feed_forward_norm=NormSpec("rmsnorm", H, 1e-5, f"l{i}.n2")) for i, m in enumerate(layers)),
        order=tuple(RunStep(i) for i in range(len(layers))),
        final_norm=NormSpec("rmsnorm", H, 1e-5, "fn"), head=HeadSpec(vocab, H, None), max_position=128)


def _toy_weights(plan, extra, seed=0):
    g = torch.Generator().manual_seed(seed)
    H, V = plan.embedding.hidden_size, plan.embedding.vocab_size
    w = {"emb": torch.randn(V, H, generator=g) * 0.5, "fn": torch.ones(H)}
    for i in range(len(plan.layers)):
        w.update({f"l{i}.n1": 1 + 0.1 * torch.randn(H, generator=g), f"l{i}.n2": torch.ones(H),
                  f"l{i}.mlp.gate_proj.weight": torch.randn(2 * H, H, generator=g) * 0.1,
                  f"l{i}.mlp.up_proj.weight": torch.randn(2 * H, H, generator=g) * 0.1,
                  f"l{i}.mlp.down_proj.weight": torch.randn(H, 2 * H, generator=g) * 0.1})
    w.update(extra(g))
    return w


def test_a_toy_mixer_with_state_is_registered_built_and_stepped():
    """No file of the package changes: the test registers the kind, builds a plan that mixes the
    toy mixer with the package's attention layer by layer, and steps it in portions.  Two
    requests interleaved must not see each other's state; portions must carry the state on."""
    from tandem_b200.config.plan import AttentionSpec, PositionSpec
    from tandem_b200.engine.core import build_executor
    from tandem_b200.engine.executor import StepEntry
    from tandem_b200.models.decoder import Decoder
    from tandem_b200.registry import register_part
    from tandem_b200.weights.loader import TensorDict

    register_part("mixer", "toy_decay", DecayMixer)
    H, V = 32, 50
    attn = AttentionSpec("attention", prefix="l1.attn", hidden_size=H, num_heads=2, num_kv_heads=1, head_dim=16,
                         scale=0.25, qk_norm=False, position=PositionSpec("rope", rotary_dim=16, theta=100.0, max_position=128))
    plan = _toy_plan(V, H, [DecaySpec(prefix="l0.mix", hidden_size=H, decay=0.7), attn, DecaySpec(prefix="l2.mix", hidden_size=H)])

    def extra(g):
        return {"l0.mix.w": torch.randn(H, H, generator=g) * 0.1, "l2.mix.w": torch.randn(H, H, generator=g) * 0.1,
                "l1.attn.q_proj.weight": torch.randn(32, H, generator=g) * 0.2, "l1.attn.k_proj.weight": torch.randn(16, H, generator=g) * 0.2,
                "l1.attn.v_proj.weight": torch.randn(16, H, generator=g) * 0.2, "l1.attn.o_proj.weight": torch.randn(H, 32, generator=g) * 0.2}

    decoder = Decoder(plan, TensorDict(_toy_weights(plan, extra)), torch.float32, "cuda")
    assert [n is not None for n in decoder.kv_needs()] == [False, True, False]
    assert [n is not None for n in decoder.state_needs()] == [True, False, True]
    ex = build_executor(decoder, page_size=8, num_pages=16, max_requests=3)
    a, b = random_tokens(1, 40, V), random_tokens(2, 27, V)
    whole_a = ex.step([StepEntry("a", a, list(range(40)))], end=["a"])
    whole_b = ex.step([StepEntry("b", b, list(range(27)))], end=["b"])
    # the same two requests in interleaved portions; a slot that is used again starts from zero state
    got_a, got_b = [], []
    ia = ib = 0
    for na, nb in ((7, 2), (2, 13), (20, 1), (11, 11)):
        entries = []
        if na:
            entries.append(StepEntry("a2", a[ia: ia + na], list(range(na))))
        if nb:
            entries.append(StepEntry("b2", b[ib: ib + nb], list(range(nb))))
        out = ex.step(entries)
        got_a.append(out[:na]), got_b.append(out[na:])
        ia, ib = ia + na, ib + nb
    assert ia == 40 and ib == 27
    torch.testing.assert_close(torch.cat(got_a), whole_a, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(torch.cat(got_b), whole_b, atol=1e-5, rtol=1e-5)
    ex.step([], end=["a2", "b2"])
    assert ex.manager.all_free()


def test_the_order_may_name_a_layer_twice_or_share_a_cache():
    """order = [0, 1, 0, 1 reading the cache of run 1]: run 2 reuses layer 0's weights with a
    cache of its own; run 3 reuses layer 1's weights and reads the keys run 1 stored."""
    from tandem_b200.config.model_config import Qwen3Config
    from tandem_b200.config.plan import RunStep
    from tandem_b200.engine.core import build_executor
    from tandem_b200.engine.executor import StepEntry
    from tandem_b200.models.decoder import Decoder
    from tandem_b200.models.qwen3 import build_plan, random_weights
    from tandem_b200.weights.loader import TensorDict

    cfg = Qwen3Config.from_dict(TINY["A"])
    weights = dict(random_weights(cfg, 5, "cpu", torch.float32, std=0.1))
    plan = replace(build_plan(cfg), order=(RunStep(0), RunStep(1), RunStep(0), RunStep(1, cache_of=1)))
    decoder = Decoder(plan, TensorDict(dict(weights)), torch.float32, "cuda")
    assert [n is not None for n in decoder.kv_needs()] == [True, True, True, False]
    ex = build_executor(decoder, page_size=4, num_pages=32, max_requests=2)
    assert sorted(ex.storage.k) == [0, 1, 2] and ex.storage.source_run[3] == 1
    tokens = random_tokens(9, 30, 512)
    whole = ex.step([StepEntry("w", tokens, list(range(30)))], end=["w"])
    parts = [ex.step([StepEntry("p", tokens[i: i + n], list(range(n)))]) for i, n in ((0, 9), (9, 2), (11, 19))]
    torch.testing.assert_close(torch.cat(parts), whole, atol=1e-5, rtol=1e-5)

    # plain: layers 0, 1, 0, then layer 1's weights with its *own earlier* keys and values
    w = {k: v.float() for k, v in weights.items()}
    d = plain.derived(TINY["A"])
    cos, sin = plain.rope_tables(d["hd"], d["theta"], 30, torch.float32)
    h = w["model.embed_tokens.weight"][torch.tensor(tokens)]
    h = plain.decoder_layer(h, w, 0, d, cos, sin)
    x1 = plain.rms_norm(h, w["model.layers.1.input_layernorm.weight"], d["eps"])  # what run 1's k, v came from
    h = plain.decoder_layer(h, w, 1, d, cos, sin)
    h = plain.decoder_layer(h, w, 0, d, cos, sin)
    p = "model.layers.1.self_attn"
    x3 = plain.rms_norm(h, w["model.layers.1.input_layernorm.weight"], d["eps"])
    q = plain.apply_rope(plain.rms_norm((x3 @ w[f"{p}.q_proj.weight"].T).view(30, d["nh"], d["hd"]), w[f"{p}.q_norm.weight"], d["eps"]), cos, sin)
    k = plain.apply_rope(plain.rms_norm((x1 @ w[f"{p}.k_proj.weight"].T).view(30, d["nkv"], d["hd"]), w[f"{p}.k_norm.weight"], d["eps"]), cos, sin)
    v = (x1 @ w[f"{p}.v_proj.weight"].T).view(30, d["nkv"], d["hd"])
    h = h + plain.attention_scores(q, k, v, None).reshape(30, -1) @ w[f"{p}.o_proj.weight"].T
    h = h + plain.swiglu(plain.rms_norm(h, w["model.layers.1.post_attention_layernorm.weight"], d["eps"]), w, "model.layers.1.mlp")
    want = plain.rms_norm(h, w["model.norm.weight"], d["eps"]) @ w["model.embed_tokens.weight"].T
    torch.testing.assert_close(whole.cpu(), want, atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_overlap_scheduling_changes_no_token(tiny_folder, dtype):
    """Launching step N before the host has read step N-1's tokens gives the tokens of the
    synchronous loop: greedy and seeded sampling, prompts cut by the budget, requests that end on a
    stop token while their next token is already in flight, a pool so small that requests are
    preempted, and a request of a single new token."""
    from tandem_b200 import EngineConfig, LLMEngine, SamplingParams

    folder = tiny_folder("B", 0.1)
    prompts = [random_tokens(80 + i, n, 1000) for i, n in enumerate([1, 9, 40, 23, 5])]

    def run(overlap, sps, **options):
        eng = LLMEngine(EngineConfig(model=folder, dtype=dtype, block_size=8, max_num_batched_tokens=16,
                                     schedule_policy="decode_first", overlap_schedule=overlap, **options))
        outs = eng.generate(prompts, sps)
        eng.cache.check()
        assert eng.cache.all_free() and eng.inflight is None
        return [(o.output_token_ids, o.finish_reason) for o in outs], eng

    greedy = [SamplingParams(max_tokens=n, **GREEDY) for n in (12, 1, 20, 7, 2)]
    sync, _ = run(False, greedy, num_kv_blocks=64)
    over, eng = run(True, greedy, num_kv_blocks=64)
    assert over == sync and eng.overlap
    # stop tokens: take tokens that the greedy run produced in the middle of two requests
    stops = [SamplingParams(max_tokens=20, temperature=0.0, ignore_eos=True, stop_token_ids=[sync[i][0][k]])
             if i in (0, 2) else SamplingParams(max_tokens=6, **GREEDY) for i, k in zip(range(5), (5, 0, 9, 0, 0))]
    sync_stop, _ = run(False, stops, num_kv_blocks=64)
    over_stop, _ = run(True, stops, num_kv_blocks=64)
    assert over_stop == sync_stop and sync_stop[0][1] == "stop" and sync_stop[2][1] == "stop"
    # seeded sampling
    drawn = [SamplingParams(max_tokens=10, temperature=0.9, top_k=50, seed=7 + i, ignore_eos=True) for i in range(5)]
    assert run(True, drawn, num_kv_blocks=64)[0] == run(False, drawn, num_kv_blocks=64)[0]
    # 10 pages of 8 tokens: five requests of up to 60 tokens do not fit, some are preempted
    small, eng = run(True, greedy, num_kv_blocks=10, max_num_seqs=5)
    assert small == sync and eng.scheduler.num_preemptions > 0


def test_graphs_captured_when_the_engine_is_built(tiny_folder):
    """``cuda_graph_capture_at_start``: every bucket is captured with requests of the engine's own, which give
    their pages back; generation then replays from its first decode step on and returns what an engine that
    captures at first use returns (float32: a replayed step gives the bits of the eager one)."""
    from tandem_b200 import EngineConfig, LLMEngine, SamplingParams

    folder = tiny_folder("B", 0.1)
    prompts = [random_tokens(700 + i, n, 1000) for i, n in enumerate([12, 3, 30])]
    sp = SamplingParams(max_tokens=10, **GREEDY)

    def build(at_start):
        return LLMEngine(EngineConfig(model=folder, dtype="float32", block_size=8, num_kv_blocks=40, max_num_seqs=6,
                                      cuda_graph_max_bs=6, cuda_graph_capture_at_start=at_start))

    early, late = build(True), build(False)
    assert set(early.graphs.captured) == {1, 2, 4, 6} and not late.graphs.captured
    assert early.cache.all_free()
    early.cache.check()
    replays_before = sum(c.replays for c in early.graphs.captured.values())
    a = [o.output_token_ids for o in early.generate(prompts, sp)]
    b = [o.output_token_ids for o in late.generate(prompts, sp)]
    assert a == b and early.cache.all_free()
    assert sum(c.replays for c in early.graphs.captured.values()) - replays_before >= 9  # every decode step was a replay
    # a pool too small for the largest bucket: that one is left for its first step
    tight = LLMEngine(EngineConfig(model=folder, dtype="float32", block_size=8, num_kv_blocks=3, max_num_seqs=6,
                                   cuda_graph_max_bs=6, cuda_graph_capture_at_start=True))
    assert set(tight.graphs.captured) == {1, 2} and tight.cache.all_free()


def test_overlap_scheduling_with_captured_steps_that_bring_prompt_portions(tmp_path):
    """A head size with which steps that bring prompt portions are replayed from CUDA graphs: tokens that
    are still on their way enter such a step on the device like any other.  Requests arrive while others
    decode (a small budget cuts their prompts).  The overlap loop and the synchronous loop batch their
    steps differently (a request that has ended is seen a step later), so in bfloat16 they may part at a
    near-tie; what is checked is that every token either loop generated is the plain implementation's
    greedy choice given the tokens before it, to within bfloat16 rounding, and that most steps with
    portions were replays."""
    from tandem_b200 import EngineConfig, LLMEngine, SamplingParams
    from tandem_b200.weights.random_init import write_random_model

    config = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=128,
                  num_attention_heads=4, num_key_value_heads=2, head_dim=64, intermediate_size=256, vocab_size=1000,
                  rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=512)
    folder = str(tmp_path / "hd64")
    write_random_model(config, folder, seed=3, dtype="bfloat16", std=0.1)
    cfg, w64 = plain.read_folder(folder, torch.float64)
    prompts = [random_tokens(300 + i, n, 1000) for i, n in enumerate([33, 9, 70, 2, 48, 17, 90, 5])]
    params = [SamplingParams(max_tokens=n, temperature=0.0, ignore_eos=True) for n in (20, 7, 12, 30, 9, 25, 6, 14)]

    def run(overlap):
        eng = LLMEngine(EngineConfig(model=folder, dtype="bfloat16", block_size=16, max_num_batched_tokens=40, num_kv_blocks=64,
                                     max_num_seqs=8, schedule_policy="decode_first", overlap_schedule=overlap), load_tokenizer=False)
        assert eng.graphs is not None and eng.graphs.mixed
        ids = [eng.add_request(p, sp) for p, sp in zip(prompts[:3], params[:3])]
        final, steps = {}, 0
        while eng.has_unfinished_requests() or len(ids) < len(prompts):
            if steps % 4 == 3 and len(ids) < len(prompts):  # the others arrive while these decode
                ids.append(eng.add_request(prompts[len(ids)], params[len(ids)]))
            for out in eng.step():
                if out.finished:
                    final[out.request_id] = out.output_token_ids
            steps += 1
        eng.cache.check()
        assert eng.cache.all_free() and eng.inflight is None
        return [final[i] for i in ids], eng

    for overlap in (False, True):
        outs, eng = run(overlap)
        for prompt, got, sp in zip(prompts, outs, params):
            assert len(got) == sp.max_tokens
            logits = plain.forward(cfg, w64, prompt + got, torch.float64)[len(prompt) - 1: -1]  # the rows that chose got[0], got[1], ...
            chosen = logits.gather(1, torch.tensor(got).unsqueeze(1)).squeeze(1)
            short = (logits.max(dim=1).values - chosen).max().item()
            assert short < 0.08, (overlap, short)  # bfloat16 logits of this model are within 0.03 of the float64 ones
        mixed = [c for k, c in eng.graphs.captured.items() if isinstance(k, tuple)]
        assert mixed and sum(c.replays for c in mixed) >= 5 and eng.graphs.mixed_fallbacks == 0


@dataclass(frozen=True)
class RoutedSpec:
    family = "feed_forward"
    kind: str = "toy_routed"
    prefix: str = ""
    hidden_size: int = 0
    experts: int = 3
    width: int = 0


class RoutedFeedForward:
    """A toy feed-forward with routing, defined here, not in the package: every token goes to the
    expert whose router logit (float32) is largest and is scaled by its softmax weight."""

    @staticmethod
    def params(spec):
        from tandem_b200.config.plan import ParamSpec, WeightSource

        out = {"router": ParamSpec((spec.experts, spec.hidden_size), (WeightSource(f"{spec.prefix}.router"),))}
        for e in range(spec.experts):
            out[f"up{e}"] = ParamSpec((spec.width, spec.hidden_size), (WeightSource(f"{spec.prefix}.e{e}.up"),))
            out[f"down{e}"] = ParamSpec((spec.hidden_size, spec.width), (WeightSource(f"{spec.prefix}.e{e}.down"),))
        return out

    def __init__(self, spec, weights, dtype, device):
        self.spec, self.w = spec, weights

    def forward(self, x, ctx):
        from tandem_b200.kernels import ops

        logits = x.float() @ self.w["router"].float().T
        gate, choice = torch.softmax(logits, -1).max(-1)
        out = torch.zeros_like(x)
        for e in range(self.spec.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():  # the package's own matrix product on the expert's rows
                h = torch.relu(ops.linear(x[rows].contiguous(), self.w[f"up{e}"]))
                out[rows] = (gate[rows, None] * ops.linear(h, self.w[f"down{e}"]).float()).to(x.dtype)
        return out


class HalfRateRotary:
    """A toy position encoding: the rotary table of the package's layout, with angles that advance
    half as fast and only over the first half of the pairs (the rest stay unrotated)."""

    def __init__(self, spec, device):
        self.rotary_dim = spec.rotary_dim
        half = spec.rotary_dim // 2
        inv = 1.0 / (spec.theta ** (torch.arange(half, dtype=torch.float32) / half))
        inv[half // 2:] = 0.0
        ang = torch.outer(0.5 * torch.arange(spec.max_position, dtype=torch.float32), inv)
        self.cos_sin = torch.cat([ang.cos(), ang.sin()], -1).contiguous().to(device)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_toy_routed_feed_forward_and_a_toy_position_encoding(dtype):
    """Registered from here, chosen layer by layer in a plan beside the package's own parts, built
    and stepped without a change to the package; portions and a mixed batch give what whole
    prompts give, and the whole prompt gives what plain torch gives."""
    from tandem_b200.config.plan import AttentionSpec, PositionSpec
    from tandem_b200.engine.core import build_executor
    from tandem_b200.engine.executor import StepEntry
    from tandem_b200.models.decoder import Decoder
    from tandem_b200.registry import register_part
    from tandem_b200.weights.loader import TensorDict

    register_part("feed_forward", "toy_routed", RoutedFeedForward)
    register_part("position", "toy_half_rate", HalfRateRotary)
    H, V, hd, nh, nkv = 64, 90, 32, 4, 2
    plan = _toy_plan(V, H, [
        AttentionSpec("attention", prefix=f"l{i}.attn", hidden_size=H, num_heads=nh, num_kv_heads=nkv, head_dim=hd,
                      scale=hd ** -0.5, qk_norm=False,
                      position=PositionSpec("toy_half_rate" if i == 0 else "rope", rotary_dim=hd, theta=50.0, max_position=128))
        for i in range(2)])
    layers = list(plan.layers)
    layers[1] = layers[1].with_slot("feed_forward", RoutedSpec(prefix="l1.moe", hidden_size=H, experts=3, width=48))
    plan = replace(plan, layers=tuple(layers))

    def extra(g):
        out = {}
        for i in range(2):
            out.update({f"l{i}.attn.q_proj.weight": torch.randn(nh * hd, H, generator=g) * 0.2,
                        f"l{i}.attn.k_proj.weight": torch.randn(nkv * hd, H, generator=g) * 0.2,
                        f"l{i}.attn.v_proj.weight": torch.randn(nkv * hd, H, generator=g) * 0.2,
                        f"l{i}.attn.o_proj.weight": torch.randn(H, nh * hd, generator=g) * 0.2})
        out["l1.moe.router"] = torch.randn(3, H, generator=g)
        for e in range(3):
            out[f"l1.moe.e{e}.up"] = torch.randn(48, H, generator=g) * 0.2
            out[f"l1.moe.e{e}.down"] = torch.randn(H, 48, generator=g) * 0.2
        return out

    weights = {k: v for k, v in _toy_weights(plan, extra, seed=3).items() if not k.startswith("l1.mlp.")}
    decoder = Decoder(plan, TensorDict(dict(weights)), dtype, "cuda")
    ex = build_executor(decoder, page_size=8, num_pages=24, max_requests=3)
    a, b = random_tokens(5, 37, V), random_tokens(6, 21, V)
    whole_a = ex.step([StepEntry("a", a, list(range(37)))], end=["a"])
    whole_b = ex.step([StepEntry("b", b, list(range(21)))], end=["b"])
    got_a, got_b, ia, ib = [], [], 0, 0
    for na, nb in ((9, 2), (2, 7), (25, 1), (1, 11)):
        out = ex.step([StepEntry("a2", a[ia: ia + na], list(range(na))), StepEntry("b2", b[ib: ib + nb], list(range(nb)))])
        got_a.append(out[:na]), got_b.append(out[na:])
        ia, ib = ia + na, ib + nb
    ex.step([], end=["a2", "b2"])
    assert ex.manager.all_free()
    cut = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.15, rtol=0.05)
    torch.testing.assert_close(torch.cat(got_a), whole_a, **cut)
    torch.testing.assert_close(torch.cat(got_b), whole_b, **cut)
    if dtype != torch.float32:
        return  # in bfloat16 a token near a routing tie may take another expert than plain float64 does

    # plain torch, whole prompt, float64
    w = {k: v.double() for k, v in weights.items()}
    T = len(a)
    h = w["emb"][torch.tensor(a)]
    pos = torch.arange(T, dtype=torch.float64)
    for i in range(2):
        x = plain.rms_norm(h, w[f"l{i}.n1"], 1e-5)
        q = (x @ w[f"l{i}.attn.q_proj.weight"].T).view(T, nh, hd)
        k = (x @ w[f"l{i}.attn.k_proj.weight"].T).view(T, nkv, hd)
        v = (x @ w[f"l{i}.attn.v_proj.weight"].T).view(T, nkv, hd)
        half = hd // 2
        inv = 1.0 / (50.0 ** (torch.arange(half, dtype=torch.float64) / half))
        if i == 0:
            inv[half // 2:] = 0.0
            ang = torch.outer(0.5 * pos, inv)
        else:
            ang = torch.outer(pos, inv)
        cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
        q, k = plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin)
        h = h + plain.attention_scores(q, k, v, None).reshape(T, -1) @ w[f"l{i}.attn.o_proj.weight"].T
        x = plain.rms_norm(h, w[f"l{i}.n2"], 1e-5)
        if i == 0:
            h = h + plain.swiglu(x, w, "l0.mlp")
        else:
            gate, choice = torch.softmax(x @ w["l1.moe.router"].T, -1).max(-1)
            y = torch.stack([gate[t] * (torch.relu(x[t] @ w[f"l1.moe.e{int(choice[t])}.up"].T) @ w[f"l1.moe.e{int(choice[t])}.down"].T)
                             for t in range(T)])
            h = h + y
    want = plain.rms_norm(h, w["fn"], 1e-5) @ w["emb"].T
    torch.testing.assert_close(whole_a.cpu().double(), want, atol=2e-4, rtol=2e-4)


def test_overlap_scheduling_under_random_workloads(tiny_folder):
    """Random prompts, lengths, stop tokens, budgets, policies and pool sizes (some so small that
    requests are preempted): the overlap loop returns what the synchronous loop returns, request
    by request, and gives every page back."""
    import random

    from tandem_b200 import EngineConfig, LLMEngine, SamplingParams

    folder = tiny_folder("A", 0.1)
    rng = random.Random(7)
    preempted = 0
    for trial in range(6):
        n = rng.randint(3, 9)
        prompts = [random_tokens(1000 * trial + i, rng.randint(1, 45), 512) for i in range(n)]
        sps = []
        for i in range(n):
            greedy = rng.random() < 0.5
            sps.append(SamplingParams(max_tokens=rng.randint(1, 24), temperature=0.0 if greedy else 0.8,
                                      top_k=-1 if greedy else 40, seed=trial * 100 + i, ignore_eos=True,
                                      stop_token_ids=[rng.randrange(512) for _ in range(rng.randint(0, 40))]))
        options = dict(block_size=rng.choice([4, 8, 16]), max_num_batched_tokens=rng.choice([8, 16, 64]),
                       schedule_policy=rng.choice(["decode_first", "prefill_first"]), max_num_seqs=rng.choice([2, 4, 8]))
        options["num_kv_blocks"] = max(-(-70 // options["block_size"]) + 1, rng.choice([6, 12, 40]))
        results = []
        for overlap in (False, True):
            eng = LLMEngine(EngineConfig(model=folder, dtype="float32", overlap_schedule=overlap, **options))
            outs = eng.generate(prompts, sps)
            results.append([(o.output_token_ids, o.finish_reason) for o in outs])
            eng.cache.check()
            assert eng.cache.all_free() and eng.inflight is None and not eng.requests
            preempted += eng.scheduler.num_preemptions
        assert results[0] == results[1], (trial, options)
    assert preempted > 0


@pytest.mark.parametrize("overlap", [False, True])
def test_a_generation_run_is_recorded_as_a_trace_that_replays(tiny_folder, tmp_path, overlap):
    """``record_steps`` writes what the scheduler really did (portions, mixed steps, a request that
    is preempted and read again) in the replay tool's format; replaying the file gives, at every
    place where a token was sampled, logits whose argmax is that token."""
    import json

    import numpy as np

    from tandem_b200 import EngineConfig, LLMEngine, SamplingParams
    from tandem_b200.engine.trace import replay

    folder = tiny_folder("A", 0.1)
    eng = LLMEngine(EngineConfig(model=folder, dtype="float32", block_size=4, num_kv_blocks=12, max_num_batched_tokens=16,
                                 schedule_policy="decode_first", overlap_schedule=overlap))
    path = str(tmp_path / "run.jsonl")
    eng.record_steps(path)
    prompts = [random_tokens(40 + i, 10, 512) for i in range(4)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=14, **GREEDY))
    need = eng.trace.close()
    assert eng.scheduler.num_preemptions > 0
    steps = [json.loads(line) for line in open(path)]
    assert any("~" in e["id"] for s in steps for e in s["entries"])  # a recomputed request under its new id
    assert all(t >= 0 for s in steps for e in s["entries"] for t in e["tokens"])  # no placeholder left
    out_dir = str(tmp_path / "logits")
    assert replay(folder, "float32", out_dir, need, open(path), page_size=4) == len(steps)
    sampled = {o.request_id: list(o.output_token_ids) for o in outs}
    position = {}  # trace id -> tokens fed so far
    checked = 0
    for s in steps:
        wanted = sum(len(e["want"]) for e in s["entries"])
        rows = np.fromfile(f"{out_dir}/{s['step']}.f32", dtype="<f4").reshape(wanted, 512) if wanted else []
        r = 0
        for e in s["entries"]:
            position[e["id"]] = position.get(e["id"], 0) + len(e["tokens"])
            for _ in e["want"]:
                k = position[e["id"]] - 10  # index of the generated token this row decides
                assert int(rows[r].argmax()) == sampled[e["id"].split("~")[0]][k]
                r += 1
                checked += 1
    assert checked >= 4 * 14
