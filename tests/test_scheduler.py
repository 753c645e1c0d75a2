"""The scheduler's decisions, driven by fake tokens without a model (CPU), in the manner of
tests/test_scheduler.py:20-81 of 12vivi/tandem."""

import pytest

from tandem_b200.cache.manager import CacheManager, KVNeed
from tandem_b200.engine.request import Request, RequestStatus
from tandem_b200.engine.scheduler import Scheduler
from tandem_b200.sampling.params import SamplingParams


def make(policy="prefill_first", pages=64, page_size=4, budget=8, max_seqs=8, max_len=256, window=None):
    cache = CacheManager([KVNeed(2, 16, window)], page_size, pages, max_seqs)
    return Scheduler(cache, max_seqs, budget, max_len, policy), cache


def req(rid, n, max_tokens=4, **kw):
    return Request(rid, list(range(1, n + 1)), SamplingParams(max_tokens=max_tokens, temperature=0.0, **kw),
                   eos_token_ids=[0])


def run_step(s, token=7):
    plan = s.schedule()
    sampled = {x.request.request_id: token for x in plan.scheduled
               if x.request.num_computed_tokens + x.num_tokens >= x.request.num_tokens}
    s.update_from_output(plan, sampled)
    return plan


def sizes(plan):
    return [(x.request.request_id, x.num_tokens) for x in plan.scheduled]


def test_prompt_is_cut_by_the_budget():
    s, cache = make(budget=8)
    s.add_request(req("a", 20))
    assert [sizes(run_step(s)) for _ in range(3)] == [[("a", 8)], [("a", 8)], [("a", 4)]]
    assert sizes(run_step(s)) == [("a", 1)]  # decoding now
    cache.check()


def test_budget_is_shared_in_arrival_order():
    s, _ = make(budget=8)
    for rid, n in (("a", 5), ("b", 5), ("c", 2)):
        s.add_request(req(rid, n))
    assert sizes(run_step(s)) == [("a", 5), ("b", 3)]
    assert sizes(run_step(s)) == [("b", 2), ("c", 2)]  # prefill_first: a (decoding) waits


def test_decode_first_mixes_and_prefill_first_does_not():
    for policy, expect in (("decode_first", [("a", 1), ("b", 7)]), ("prefill_first", [("b", 8)])):
        s, _ = make(policy=policy, budget=8)
        s.add_request(req("a", 3, max_tokens=10))
        run_step(s)
        s.add_request(req("b", 12))
        assert sizes(run_step(s)) == expect


def test_prefill_first_falls_back_to_decoding_when_nothing_fits():
    s, _ = make(pages=4, page_size=4, budget=16)
    s.add_request(req("a", 10, max_tokens=3))  # 3 pages
    run_step(s)
    s.add_request(req("b", 8))  # needs 2 pages, 1 free: stays waiting at the head
    plan = run_step(s)
    assert sizes(plan) == [("a", 1)] and [r.request_id for r in s.waiting] == ["b"]


def test_max_num_seqs_limits_admission():
    s, _ = make(max_seqs=2, budget=64)
    for rid in "abc":
        s.add_request(req(rid, 3))
    assert sizes(run_step(s)) == [("a", 3), ("b", 3)] and len(s.waiting) == 1


def test_finishing_by_length_eos_and_stop_token():
    s, cache = make(budget=64)
    s.add_request(req("a", 3, max_tokens=2))
    run_step(s), run_step(s)
    assert not s.has_unfinished() and cache.all_free()
    s.add_request(r := req("b", 3, max_tokens=9))
    run_step(s, token=0)  # eos
    assert r.status is RequestStatus.FINISHED_STOPPED and r.finish_reason == "stop"
    s.add_request(r := req("c", 3, max_tokens=9, ignore_eos=True, stop_token_ids=[5]))
    run_step(s, token=0)
    assert not r.finished
    run_step(s, token=5)
    assert r.finish_reason == "stop" and r.output_token_ids == [0, 5] and cache.all_free()


def test_max_model_len_ends_a_request():
    s, _ = make(max_len=6, budget=64)
    s.add_request(r := req("a", 4, max_tokens=50))
    while s.has_unfinished():
        run_step(s)
    assert r.finish_reason == "length" and r.num_tokens == 6
    with pytest.raises(ValueError):
        s.add_request(req("b", 6))


def test_pages_run_out_youngest_is_preempted_and_recomputed():
    # 6 pages of 4 tokens; two requests of 8 + up to 10 tokens cannot both grow to the end
    s, cache = make(policy="decode_first", pages=6, page_size=4, budget=32)
    a, b = req("a", 8, max_tokens=10), req("b", 8, max_tokens=10)
    s.add_request(a), s.add_request(b)
    preempted = []
    steps = 0
    while s.has_unfinished():
        plan = run_step(s)
        preempted += [r.request_id for r in plan.preempted]
        cache.check()
        steps += 1
        assert steps < 200
    assert preempted and set(preempted) == {"b"}  # the oldest request is never the victim
    assert s.num_preemptions == len(preempted) and b.num_preemptions == len(preempted)
    assert a.num_output_tokens == 10 and b.num_output_tokens == 10  # generated tokens survive recompute
    assert cache.all_free()


def test_preempted_request_goes_to_the_front_and_no_admission_in_that_step():
    s, cache = make(policy="decode_first", pages=4, page_size=4, budget=32)
    a, b = req("a", 8, max_tokens=20), req("b", 8, max_tokens=20)
    s.add_request(a), s.add_request(b)
    run_step(s)  # both admitted: 2 + 2 pages, all full
    s.add_request(req("c", 2))
    plan = run_step(s)  # both need a third page: b, the youngest, is preempted for a
    assert [r.request_id for r in plan.preempted] == ["b"] and sizes(plan) == [("a", 1)]
    assert [r.request_id for r in s.waiting] == ["b", "c"]
    assert b.num_computed_tokens == 0 and b.num_output_tokens == 1 and not cache.has("b")


def test_a_request_alone_always_fits():
    s, cache = make(pages=3, page_size=4, budget=64, max_len=100)
    assert s.max_model_len == 12  # the pool caps the length of a request
    s.add_request(r := req("a", 5, max_tokens=50))
    while s.has_unfinished():
        run_step(s)
    assert r.finish_reason == "length" and r.num_tokens == 12 and cache.all_free()
    with pytest.raises(ValueError):
        s.add_request(req("b", 12))


def test_abort_releases_pages():
    s, cache = make()
    s.add_request(a := req("a", 6))
    s.add_request(b := req("b", 6))
    run_step(s)
    s.finish_request(a, RequestStatus.FINISHED_ABORTED)
    s.finish_request(b, RequestStatus.FINISHED_ABORTED)
    assert a.finish_reason == "abort" and not s.has_unfinished() and cache.all_free()


def test_windowed_request_outlives_the_pool():
    s, cache = make(pages=4, page_size=4, budget=8, window=6, max_len=16)
    s.add_request(r := req("a", 5, max_tokens=11))
    while s.has_unfinished():
        run_step(s)
        cache.check()
    assert r.num_tokens == 16 and cache.all_free()


# ----------------------------------------------------------------------------- overlap scheduling
def overlap_step(s, inflight, tokens):
    """One call of the engine's overlap loop with fake tokens: schedule and book step N, then
    resolve step N-1 (``tokens``: request id -> token for the step being resolved)."""
    plan = s.schedule()
    plan.promised = [x.request.request_id for x in plan.scheduled
                     if x.request.num_computed_tokens + x.num_tokens >= x.request.num_tokens]
    if not plan.is_empty:
        s.book_launch(plan)
    if inflight is not None:
        s.deliver_tokens(inflight, {rid: tokens.get(rid, 7) for rid in inflight.promised})
    return plan


def test_overlap_books_a_placeholder_and_fills_it_one_step_later():
    from tandem_b200.engine.request import PLACEHOLDER

    s, cache = make(budget=8)
    a = req("a", 5, max_tokens=3)
    s.add_request(a)
    p0 = overlap_step(s, None, {})
    assert sizes(p0) == [("a", 5)] and a.token_ids[5:] == [PLACEHOLDER] and a.output_token_ids == [] and a.num_known_outputs == 0
    p1 = overlap_step(s, p0, {"a": 11})  # decodes with its token still on the way, then learns it
    assert sizes(p1) == [("a", 1)] and a.token_ids[5:] == [11, PLACEHOLDER] and a.output_token_ids == [11]
    p2 = overlap_step(s, p1, {"a": 12})
    assert sizes(p2) == [("a", 1)] and a.token_ids[5:] == [11, 12, PLACEHOLDER] and a.num_output_tokens == 3
    p3 = overlap_step(s, p2, {"a": 13})  # the third token is the last it may produce: not scheduled again
    assert p3.is_empty and a.finished and a.finish_reason == "length" and a.output_token_ids == [11, 12, 13]
    assert a.token_ids == [1, 2, 3, 4, 5, 11, 12, 13]
    assert not s.has_unfinished() and cache.all_free()


def test_overlap_drops_the_token_launched_after_an_end_token():
    s, cache = make(budget=8)
    a, b = req("a", 3, max_tokens=8), req("b", 4, max_tokens=8)
    s.add_request(a)
    s.add_request(b)
    p0 = overlap_step(s, None, {})
    p1 = overlap_step(s, p0, {"a": 0, "b": 5})  # a's first token is its end token (0), found after p1 was launched
    assert ("a", 1) in sizes(p1) and a.finished and a.finish_reason == "stop" and a.output_token_ids == [0]
    p2 = overlap_step(s, p1, {"a": 9, "b": 6})  # p1's token for a is dropped
    assert sizes(p2) == [("b", 1)] and a.output_token_ids == [0] and b.output_token_ids[:2] == [5, 6]
    cache.check()


def test_overlap_resolves_first_when_pages_are_short():
    """The step in flight is read first only when a running request may have to give way: when the
    running requests' next shares need more pages than are free.  An empty line, a full pool whose
    requests still have room in their last pages, and waiting requests (which wait, and take
    nobody's pages) do not count."""
    s, cache = make(pages=4, page_size=4, budget=16)
    assert not s.may_preempt()  # nobody is running
    a, b = req("a", 6, max_tokens=8), req("b", 5, max_tokens=8)
    s.add_request(a)
    s.add_request(b)
    p0 = overlap_step(s, None, {})  # both prompts: 2 pages each, the pool is full
    assert sizes(p0) == [("a", 6), ("b", 5)] and cache.free_pages(0) == 0
    s.add_request(req("c", 3, max_tokens=2))  # waits; it can take nobody's pages
    assert not s.may_preempt()  # tokens 7 and 6 fit into the pages held
    p1 = overlap_step(s, p0, {"a": 11, "b": 21})
    assert sizes(p1) == [("a", 1), ("b", 1)] and not s.may_preempt()  # a's 8th token still fits
    p2 = overlap_step(s, p1, {"a": 12, "b": 22})
    assert s.may_preempt()  # a's 9th token begins a page and none is free
    s2, _ = make(pages=64, page_size=4, budget=8)
    s2.add_request(req("a", 6, max_tokens=8))
    overlap_step(s2, None, {})
    assert not s2.may_preempt()


@pytest.mark.parametrize("seed", range(12))
def test_the_overlap_loop_under_random_requests_and_tight_pools(seed):
    """The engine's overlap loop with fake tokens: pools of a few pages, windows, both policies, requests
    that arrive while others run and end by length, by an end token or by a stop token.  The step in flight
    is read first exactly when ``may_preempt`` says so; no request is ever preempted with a token on its way
    (the scheduler raises if one would be), no page is lost, and every request ends."""
    import random

    rnd = random.Random(seed)
    page, pages = rnd.choice([2, 4, 8]), rnd.randint(6, 14)
    window = rnd.choice([None, None, 3 * page])
    s, cache = make(policy=rnd.choice(["prefill_first", "decode_first"]), pages=pages, page_size=page,
                    budget=rnd.choice([4, 8, 16]), max_seqs=rnd.randint(2, 5), max_len=pages * page, window=window)
    todo = [req(f"r{i}", rnd.randint(1, max(1, pages * page // 3)), max_tokens=rnd.randint(1, 12),
                **({"stop_token_ids": [5]} if i % 3 == 0 else {})) for i in range(14)]
    inflight, steps, early_reads = None, 0, 0

    def deliver(plan):
        tokens = {rid: rnd.choice([0, 5, 7, 8, 9, 11]) if rnd.random() < 0.25 else 7 for rid in plan.promised}
        s.deliver_tokens(plan, tokens)

    while todo or s.has_unfinished() or inflight is not None:
        if todo and (steps % 3 == 0 or not s.has_unfinished()):
            s.add_request(todo.pop(0))
        if inflight is not None and s.may_preempt():
            deliver(inflight)
            inflight = None
            early_reads += 1
        plan = s.schedule()  # raises if a request with a token on its way had to give way
        plan.promised = [x.request.request_id for x in plan.scheduled
                         if x.request.num_computed_tokens + x.num_tokens >= x.request.num_tokens]
        launched = None
        if not plan.is_empty:
            s.book_launch(plan)
            launched = plan
        else:
            assert inflight is not None or plan.preempted or not s.has_unfinished(), "nothing could be placed"
        previous, inflight = inflight, launched
        if previous is not None:
            deliver(previous)
        cache.check()
        steps += 1
        assert steps < 2000
    assert cache.all_free() and not s.running and not s.waiting


def test_a_prompt_that_preempts_itself_is_reported_and_not_admitted_again_in_that_step():
    """prefill_first: the prompt pass comes out empty because the only request reading its prompt
    had to give way itself (a decoding request holds the rest of the pool and is not in that
    pass's line).  The step falls back to decoding; it still reports the preemption and admits
    nobody, so the request is not read from the start again within the same call."""
    s, cache = make(policy="prefill_first", pages=6, page_size=4, budget=8, max_len=24)
    d = req("d", 10, max_tokens=12)
    s.add_request(d)
    run_step(s), run_step(s), run_step(s)  # d: 8 + 2 prompt tokens, then decoding; it holds 3 pages
    assert d.is_decoding
    p = req("p", 14, max_tokens=2)
    s.add_request(p)
    assert sizes(run_step(s)) == [("p", 8)]  # 2 more pages; one page is left
    plan = run_step(s)  # p needs 2 more pages for its last 6 tokens: it is the whole line of the prompt pass
    assert [r.request_id for r in plan.preempted] == ["p"] and sizes(plan) == [("d", 1)]
    assert [r.request_id for r in s.waiting] == ["p"] and not cache.has("p") and p.num_computed_tokens == 0
    cache.check()
    steps = 0
    while s.has_unfinished():
        run_step(s)
        cache.check()
        steps += 1
        assert steps < 100
    assert d.num_output_tokens == 12 and p.num_output_tokens == 2 and cache.all_free()


def test_sampling_params_are_checked_in_words():
    for bad in (dict(max_tokens=0), dict(temperature=-0.1), dict(top_p=0.0), dict(top_p=1.5), dict(min_p=2.0), dict(stop=[""])):
        with pytest.raises(ValueError, match="SamplingParams"):
            SamplingParams(**bad)
    sp = SamplingParams(stop="END", stop_token_ids=(3, 4))
    assert sp.stop == ["END"] and sp.stop_token_ids == [3, 4] and not sp.greedy
    assert SamplingParams(temperature=0.0).greedy and SamplingParams(stop=None).stop == []


class ByteTokenizer:
    """Token = one byte of UTF-8; ids 256 and up are special tokens."""

    def decode(self, ids, skip_special_tokens=True):
        data = bytes(i for i in ids if i < 256)
        extra = "" if skip_special_tokens else "".join(f"<{i}>" for i in ids if i >= 256)
        return data.decode("utf-8", errors="replace") + extra


def test_text_grows_token_by_token_and_stops_at_a_stop_string():
    from tandem_b200.engine.text import OutputText

    text = "héllo wörld — END of it"
    ids = list(text.encode("utf-8"))
    t = OutputText(ByteTokenizer(), stop=["END", "zzz"])
    grown = ""
    for n in range(1, len(ids) + 1):
        delta = t.feed(ids[:n], final=False)
        assert "\ufffd" not in delta  # a character cut in two is held back until it is whole
        grown += delta
        if t.stopped:
            break
    assert t.stopped and grown == t.text == "héllo wörld — " and n == len("héllo wörld — END".encode("utf-8"))
    assert t.feed(ids, final=True) == ""  # nothing more after the stop
    whole = OutputText(ByteTokenizer())
    assert "".join(whole.feed(ids[:n], final=n == len(ids)) for n in range(1, len(ids) + 1)) == text
