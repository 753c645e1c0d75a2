"""The cache manager: which pages and which state slot each live request holds.

Runs of the model plan that keep keys and values are sorted into *groups* by what they need:
the shape of a token's entry (kv heads, head size) and how long it is kept (all keys, or a
window of them).  Each group has a page pool of its own and a block table per request; all runs
of a group share the table (each has its own storage behind the same page numbers).  Beside the
pages, every request holds one slot of the fixed-size state tensors for as long as it lives,
whether or not any mixer of the model declares such state.

Token p of a request lives in page ``table[p // page_size]`` at offset ``p % page_size``
(python/tandem/executor/forward_context.py:61).  Pages are taken when a step is about to run
(``grow``), given back when the request ends (``end``), and, in a windowed group, as soon as
the window of the request's next query has passed them; a released entry of the table is -1.

This file is bookkeeping only (no tensors); ``tandem_b200.cache.storage`` holds the memory.
12vivi/tandem has one group and no state slots (python/tandem/scheduler/scheduler.py:130-139,
191-204; python/tandem/cache/kv_cache.py:6-34).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

from tandem_b200.cache.pages import OutOfPages, PagePool, SlotPool


def cdiv(a: int, b: int) -> int:
    return -(-a // b)


@dataclass(frozen=True)
class KVNeed:
    """What one run of the plan stores per token."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None  # keys kept behind the newest one, itself included; None: all

    @property
    def group_key(self) -> tuple:
        return (self.num_kv_heads, self.head_dim, self.window)


@dataclass
class Group:
    key: tuple
    runs: list  # run indices (positions in ModelPlan.order) that store into this group
    pool: PagePool
    window: Optional[int]
    tables: dict = field(default_factory=dict)  # request id -> list of page ids (-1: given back)


@dataclass
class Live:
    slot: int
    num_tokens: int = 0  # tokens whose entries are stored


class CacheManager:
    def __init__(self, needs: Sequence[Optional[KVNeed]], page_size: int, num_pages: int, max_requests: int) -> None:
        """``needs[r]`` is what run r stores (None: nothing of its own).  Every group gets
        ``num_pages`` pages of ``page_size`` tokens."""
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.num_pages = num_pages
        self.groups: list[Group] = []
        self.group_of_run: dict[int, int] = {}
        by_key: dict[tuple, int] = {}
        for run, need in enumerate(needs):
            if need is None:
                continue
            if need.group_key not in by_key:
                by_key[need.group_key] = len(self.groups)
                self.groups.append(Group(need.group_key, [], PagePool(num_pages), need.window))
            g = by_key[need.group_key]
            self.groups[g].runs.append(run)
            self.group_of_run[run] = g
        self.slots = SlotPool(max_requests)
        self.live: dict[str, Live] = {}

    # ------------------------------------------------------------------ requests
    def begin(self, request_id: str) -> int:
        """Admit a request: it gets a state slot (returned) and empty block tables."""
        if request_id in self.live:
            raise ValueError(f"request {request_id!r} is already live")
        slot = self.slots.acquire()
        self.live[request_id] = Live(slot)
        for g in self.groups:
            g.tables[request_id] = []
        return slot

    def end(self, request_id: str) -> None:
        """Give back everything the request holds."""
        live = self.live.pop(request_id)
        for g in self.groups:
            g.pool.release([p for p in g.tables.pop(request_id) if p >= 0])
        self.slots.release(live.slot)

    def has(self, request_id: str) -> bool:
        return request_id in self.live

    def num_tokens(self, request_id: str) -> int:
        return self.live[request_id].num_tokens

    def slot(self, request_id: str) -> int:
        return self.live[request_id].slot

    def table(self, group: int, request_id: str) -> list:
        return self.groups[group].tables[request_id]

    # ------------------------------------------------------------------ pages
    def _first_needed_page(self, g: Group, start: int) -> int:
        """Index of the first page that a query at position ``start`` (or later) still reads."""
        if g.window is None:
            return 0
        return max(0, start - g.window + 1) // self.page_size

    def pages_short(self, request_id: str, total_tokens: int) -> int:
        """How many pages are lacking, over all groups, to store ``total_tokens`` tokens of the
        request (0: ``grow`` will succeed).  Counts pages that ``grow`` would first give back."""
        live = self.live[request_id]
        short = 0
        for g in self.groups:
            table = g.tables[request_id]
            first = self._first_needed_page(g, live.num_tokens)
            freed = sum(1 for p in table[:first] if p >= 0)
            need = cdiv(total_tokens, self.page_size) - len(table)
            short += max(0, need - (g.pool.num_free + freed))
        return short

    def pages_to_grow(self, request_id: str, total_tokens: int) -> list:
        """Per group, the pages that ``grow(request_id, total_tokens)`` would take from the pool beyond
        those it first gives back (negative: it gives back more than it takes)."""
        live = self.live[request_id]
        out = []
        for g in self.groups:
            table = g.tables[request_id]
            first = self._first_needed_page(g, live.num_tokens)
            freed = sum(1 for p in table[:first] if p >= 0)
            out.append(max(0, cdiv(total_tokens, self.page_size) - len(table)) - freed)
        return out

    def grow(self, request_id: str, total_tokens: int) -> bool:
        """Make room for the request to hold ``total_tokens`` tokens.  First gives back, in the
        windowed groups, the pages that the request's next query no longer reads.  Takes pages
        in every group or in none: returns False, with nothing taken, if any group is short."""
        live = self.live[request_id]
        if total_tokens < live.num_tokens:
            raise ValueError("a request cannot shrink")
        for g in self.groups:
            table = g.tables[request_id]
            first = self._first_needed_page(g, live.num_tokens)
            passed = [i for i in range(min(first, len(table))) if table[i] >= 0]
            g.pool.release([table[i] for i in passed])
            for i in passed:
                table[i] = -1
        want = [cdiv(total_tokens, self.page_size) - len(g.tables[request_id]) for g in self.groups]
        if any(n > g.pool.num_free for n, g in zip(want, self.groups)):
            return False
        for n, g in zip(want, self.groups):
            if n > 0:
                g.tables[request_id].extend(g.pool.allocate(n))
        return True

    def commit(self, request_id: str, num_new: int) -> None:
        """The step that stored ``num_new`` more tokens of the request has been issued."""
        live = self.live[request_id]
        live.num_tokens += num_new
        for g in self.groups:
            if live.num_tokens > len(g.tables[request_id]) * self.page_size:
                raise RuntimeError(f"request {request_id!r} holds more tokens than its pages can store")

    def slot_index(self, group: int, request_id: str, position: int) -> int:
        """Flat index of a token's entry: page * page_size + offset."""
        page = self.groups[group].tables[request_id][position // self.page_size]
        if page < 0:
            raise RuntimeError(f"position {position} of {request_id!r} lies in a page that was given back")
        return page * self.page_size + position % self.page_size

    # ------------------------------------------------------------------ accounting
    def free_pages(self, group: int = 0) -> int:
        return self.groups[group].pool.num_free

    def all_free(self) -> bool:
        return all(g.pool.num_free == g.pool.num_pages for g in self.groups) and \
            self.slots.num_free == self.slots.num_slots

    def check(self) -> None:
        """Every page is either free or held by exactly one table entry (no page lost or held
        twice).  Raises AssertionError otherwise."""
        for gi, g in enumerate(self.groups):
            held = [p for t in g.tables.values() for p in t if p >= 0]
            assert len(held) == len(set(held)), f"group {gi}: a page is in two tables"
            assert len(held) + g.pool.num_free == g.pool.num_pages, f"group {gi}: a page is lost"
            for p in held:
                assert g.pool.holders(p) == 1, f"group {gi}: page {p} has {g.pool.holders(p)} holders"
        assert len(self.live) + self.slots.num_free == self.slots.num_slots, "a state slot is lost"


__all__ = ["CacheManager", "KVNeed", "OutOfPages", "cdiv"]
