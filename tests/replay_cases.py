"""Builders of replay traces: the same requests cut into steps in four ways.

A trace is a list of steps in the format ``bin/trace_run`` reads:
``{"step": i, "entries": [{"id", "tokens", "want"}], "end": [ids]}``.  Every builder asks for the
logits of every position it feeds, so that ``collect`` can put them back together per request
and compare whole sequences with the plain implementation.
"""

from __future__ import annotations


def whole(requests: dict) -> list:
    """Each request alone, in one step."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def tail_one_by_one(requests: dict, tail: int = 32) -> list:
    """Most of a request in one step, then its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        cuts = [head] + [1] * (len(toks) - head)
        steps += _cut(rid, toks, cuts, len(steps))
    return steps


def changing_portions(requests: dict, sizes=(7, 2, 13, 2, 5, 3, 2, 21, 2, 9, 4, 2, 16)) -> list:
    """Portions of changing size, down to two tokens (a lone last token stays one)."""
    steps = []
    for k, (rid, toks) in enumerate(requests.items()):
        cuts, i, left = [], k, len(toks)
        while left:
            n = min(sizes[i % len(sizes)], left)
            if left - n == 1:  # do not leave a portion of one token behind, unless nothing else fits
                n = left if n + 1 <= 2 * max(sizes) else n
            cuts.append(n)
            left -= n
            i += 1
        steps += _cut(rid, toks, cuts, len(steps))
    return steps


def _cut(rid, toks, cuts, first_step) -> list:
    steps, at = [], 0
    for j, n in enumerate(cuts):
        last = at + n == len(toks)
        steps.append({"step": first_step + j, "entries": [{"id": rid, "tokens": toks[at: at + n], "want": list(range(n))}],
                      "end": [rid] if last else []})
        at += n
    return steps


def mixed(requests: dict, live: int = 4, portion: int = 11, decode_after: float = 0.6) -> list:
    """Up to ``live`` requests at a time in one batch per step: each request reads the first
    ``decode_after`` of its tokens in portions of changing size and the rest one token a step, so
    portions of some requests run beside single tokens of others; a request that ends is replaced
    by the next one, whose pages are the ones just given back when the pool is small."""
    order = list(requests.items())
    waiting = list(range(len(order)))
    at = {}
    active: list = []
    steps = []
    while waiting or active:
        while waiting and len(active) < live:
            i = waiting.pop(0)
            active.append(i)
            at[i] = 0
        entries, ended = [], []
        for slot, i in enumerate(list(active)):
            rid, toks = order[i]
            if (len(steps) + slot) % 5 == 4 and len(active) > 1:
                continue  # a request may sit a step out and go on later
            prompt_part = max(2, int(len(toks) * decode_after))
            if at[i] < prompt_part:
                n = min(max(2, (portion * (slot + 1) + len(steps) * 3) % (2 * portion)), prompt_part - at[i])
                if prompt_part - at[i] - n == 1:
                    n += 1
            else:
                n = 1
            n = min(n, len(toks) - at[i])
            entries.append({"id": rid, "tokens": toks[at[i]: at[i] + n], "want": list(range(n))})
            at[i] += n
            if at[i] == len(toks):
                ended.append(i)
        for i in ended:
            active.remove(i)
        steps.append({"step": len(steps), "entries": entries, "end": [order[i][0] for i in ended]})
    return steps


def collect(steps: list, outputs: dict) -> dict:
    """outputs: step number -> array [wanted, vocab].  Returns request id -> list of rows in
    position order (every builder above wants every position it feeds)."""
    per_request: dict = {}
    for st in steps:
        if not any(e["want"] for e in st["entries"]):
            continue
        rows = outputs[st["step"]]
        r = 0
        for e in st["entries"]:
            for _ in e["want"]:
                per_request.setdefault(e["id"], []).append(rows[r])
                r += 1
        assert r == len(rows), (st["step"], r, len(rows))
    return per_request


def tokens_needed(steps: list, round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held, peak = {}, 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return peak


class PageLog:
    """Every page number the pools hand out, and how often a page went to a new holder while
    another request was live (its keys lie beside pages that are being read)."""

    def __init__(self, manager) -> None:
        self.handed: dict = {}
        self.reused_beside_live = 0
        for g, group in enumerate(manager.groups):
            group.pool.allocate = self._wrap(group.pool.allocate, g, manager)

    def _wrap(self, allocate, g, manager):
        def logged(n):
            ids = allocate(n)
            for i in ids:
                self.handed[(g, i)] = self.handed.get((g, i), 0) + 1
                if self.handed[(g, i)] > 1 and len(manager.live) > 1:
                    self.reused_beside_live += 1
            return ids

        return logged

    @property
    def pages_reused(self) -> int:
        return sum(1 for n in self.handed.values() if n > 1)


def pages_handed_twice(steps: list, page_size: int, num_pages: int) -> tuple:
    """The trace run through the cache manager's bookkeeping alone (no device): how many pages of
    a pool of ``num_pages`` go to a second holder, and how many of those while another request is
    live.  Raises if the pool cannot hold the trace."""
    from tandem_b200.cache.manager import CacheManager, KVNeed

    m = CacheManager([KVNeed(1, 16, None)], page_size, num_pages, 64)
    handed, beside_live = {}, 0
    for st in steps:
        for e in st["entries"]:
            rid = e["id"]
            if not m.has(rid):
                m.begin(rid)
            held = len(m.table(0, rid))
            if not m.grow(rid, m.num_tokens(rid) + len(e["tokens"])):
                raise RuntimeError(f"step {st['step']}: the pool of {num_pages} pages is too small")
            for page in m.table(0, rid)[held:]:
                handed[page] = handed.get(page, 0) + 1
                beside_live += handed[page] > 1 and len(m.live) > 1
            m.commit(rid, len(e["tokens"]))
        for rid in st["end"]:
            m.end(rid)
    return sum(1 for n in handed.values() if n > 1), beside_live
