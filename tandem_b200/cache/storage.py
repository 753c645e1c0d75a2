"""Device memory behind the cache manager's page numbers and state slots.

A *cache user* is one mixer in one run of the plan; users are numbered in running order.  Per
user that stores keys and values: K and V tensors [pages, kv heads, page_size, head_dim] in
the model dtype, so one (page, kv head) tile is a contiguous block (16 x 128 bfloat16 = 4 KiB)
that a bulk copy moves at once.  12vivi/tandem keeps [pages * page_size, kv heads, head_dim]
(python/tandem/cache/kv_cache.py:9-29).  Per user whose mixer declares state: a tensor
[max requests + 1, *shape]; the last row is scratch for rows that pad a captured batch.  A user
that reads another user's cache gets that user's tensors.
"""

from __future__ import annotations

from typing import Optional, Sequence

import torch

from tandem_b200.cache.manager import CacheManager, KVNeed
from tandem_b200.parts.base import KVView, StateNeed, StepContext


class CacheStorage:
    def __init__(self, manager: CacheManager, kv_needs: Sequence[Optional[KVNeed]], cache_of: Sequence[Optional[int]],
                 state_needs: Sequence[Optional[StateNeed]], dtype: torch.dtype, device,
                 users: Optional[Sequence[tuple]] = None) -> None:
        """``users[u]`` = (run, slot name) of cache user u; default: one user per run, slot "mixer"."""
        self.manager = manager
        users = list(users) if users is not None else [(r, "mixer") for r in range(len(kv_needs))]
        self._user_of = {key: u for u, key in enumerate(users)}
        self._users_of_run: dict = {}
        for u, (run, _) in enumerate(users):
            self._users_of_run.setdefault(run, []).append(u)
        self.k: dict[int, torch.Tensor] = {}
        self.v: dict[int, torch.Tensor] = {}
        self.state: dict[int, torch.Tensor] = {}
        self.source_run: dict[int, int] = {}
        ps, pages = manager.page_size, manager.num_pages
        for run, need in enumerate(kv_needs):
            if need is None:
                continue
            shape = (pages, need.num_kv_heads, ps, need.head_dim)
            self.k[run] = torch.zeros(shape, dtype=dtype, device=device)
            self.v[run] = torch.zeros(shape, dtype=dtype, device=device)
            self.source_run[run] = run
        for run, other in enumerate(cache_of):
            if other is not None:
                if other not in self.k:
                    raise ValueError(f"run {run} reads the cache of run {other}, which stores none")
                self.source_run[run] = other
        for run, need in enumerate(state_needs):
            if need is not None:
                self.state[run] = torch.zeros((manager.slots.num_slots + 1,) + tuple(need.shape), dtype=need.dtype,
                                              device=device)
        self.scratch_slot = manager.slots.num_slots  # the state row of no request

    def user(self, run: int, mixer=None) -> int:
        """The cache user that ``mixer`` is in run ``run`` (None: the run's only mixer)."""
        if mixer is not None:
            return self._user_of[(run, getattr(mixer, "slot_name", "mixer"))]
        users = self._users_of_run.get(run, [])
        if len(users) != 1:
            raise RuntimeError(f"run {run} has {len(users)} mixers: each has to name itself, ctx.kv(self) / ctx.state(self)")
        return users[0]

    @property
    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for d in (self.k, self.v, self.state) for t in d.values())

    def view(self, run: int, ctx: StepContext) -> KVView:
        src = self.source_run[run]
        table, slots = ctx.tables[self.manager.group_of_run[src]]
        return KVView(self.k[src], self.v[src], table, slots, self.manager.page_size, writable=src == run)

    def reset_state(self, slot: int) -> None:
        """A newly admitted request starts from zero state."""
        for t in self.state.values():
            t[slot].zero_()
