"""Continuous batching with chunked prefill under a token budget.

The state machine of python/tandem/scheduler/scheduler.py:216-288,364-407 without its prefix
cache, host tier and short-prefill lane:

* two queues, ``waiting`` (first in, first out) and ``running``;
* each step has ``max_num_batched_tokens`` tokens to give; a request takes
  ``min(tokens it still lacks, budget left)``, so a prompt is cut into portions wherever the
  budget ends;
* ``prefill_first``: while anything waits or is still reading its prompt, a step carries no
  decoding request (falling back to a decode step if nothing could be prefilled);
  ``decode_first``: every decoding request first, one token each, then prompt portions, then
  admissions, all in one mixed step;
* admission in arrival order while the budget, ``max_num_seqs`` and the pages allow; a request
  that does not fit stays at the head of the queue and nothing behind it overtakes it.

When pages run out for a running request, the request that is last in this step's order (the
youngest, not yet scheduled) is preempted: everything it holds is given back, its computed-token
count returns to zero, and it goes to the *front* of the waiting queue to be recomputed later,
its generated tokens included.  A step that preempted admits nobody.  Because no request may be
longer than one group's whole pool (``token_capacity``), the oldest request can always finish,
so the queue always drains.

Overlap scheduling (scheduler.py:409-469 of the reference): the engine may launch step N before
the tokens of step N-1 have reached the host.  ``on_launch`` books a launched step at once, with a
placeholder for every token it will produce; ``update_resolved`` fills the placeholders in one
step later.  A request that turns out to have ended (its token was an end token, or it was
aborted) may already sit in the next launched step: that step's token for it is dropped.  A
request whose token in flight is the last it may produce is not scheduled again.  The engine
resolves the step in flight *before* it schedules whenever pages are so short that a preemption
is possible (``may_preempt``), so a preempted request never carries a placeholder.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field

from tandem_b200.cache.manager import CacheManager
from tandem_b200.engine.request import PLACEHOLDER, Request, RequestStatus


@dataclass
class ScheduledRequest:
    request: Request
    num_tokens: int  # tokens this step computes for it


@dataclass
class StepPlan:
    scheduled: list = field(default_factory=list)
    preempted: list = field(default_factory=list)

    @property
    def is_empty(self) -> bool:
        return not self.scheduled

    @property
    def num_tokens(self) -> int:
        return sum(s.num_tokens for s in self.scheduled)


class Scheduler:
    def __init__(self, cache: CacheManager, max_num_seqs: int, max_num_batched_tokens: int, max_model_len: int,
                 policy: str = "prefill_first") -> None:
        if policy not in ("decode_first", "prefill_first"):
            raise ValueError(f"unknown scheduling policy {policy!r}")
        self.policy = policy
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        # a request alone must fit into the pool, or preemption could never help it
        self.token_capacity = cache.num_pages * cache.page_size
        self.max_model_len = min(max_model_len, self.token_capacity)
        self.waiting: deque = deque()
        self.running: list = []
        self.num_preemptions = 0

    # ------------------------------------------------------------------ queue
    def add_request(self, req: Request) -> None:
        if req.num_prompt_tokens >= self.max_model_len:
            raise ValueError(f"prompt has {req.num_prompt_tokens} tokens; at most {self.max_model_len - 1} fit "
                             f"(max_model_len and the cache pool of {self.token_capacity} tokens)")
        req.status = RequestStatus.WAITING
        self.waiting.append(req)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def finish_request(self, req: Request, status: RequestStatus) -> None:
        """Finish a request from outside the step loop (abort)."""
        if req.finished:
            return
        if req in self.running:
            self.running.remove(req)
        elif req in self.waiting:
            self.waiting.remove(req)
        self._release(req)
        req.status = status
        req.finish_time = time.monotonic()

    # ------------------------------------------------------------------ pages
    def _release(self, req: Request) -> None:
        if self.cache.has(req.request_id):
            self.cache.end(req.request_id)

    def _preempt(self, req: Request) -> None:
        self._release(req)
        req.num_computed_tokens = 0
        req.status = RequestStatus.WAITING
        req.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(req)

    # ------------------------------------------------------------------ schedule
    def schedule(self) -> StepPlan:
        if self.policy == "prefill_first" and (self.waiting or any(not r.is_decoding for r in self.running)):
            plan = self._schedule(decodes=False)
            if not plan.is_empty:
                return plan
        return self._schedule(decodes=True)

    def _schedule(self, decodes: bool) -> StepPlan:
        plan = StepPlan()
        budget = self.max_num_batched_tokens
        order = ([r for r in self.running if r.is_decoding and not self._awaiting_last_token(r)] if decodes else []) + \
                [r for r in self.running if not r.is_decoding]

        # 1) running requests: decoding ones first, then prompt portions
        i = 0
        while i < len(order) and budget > 0:
            req = order[i]
            n = min(req.num_tokens - req.num_computed_tokens, budget)
            if n <= 0:
                i += 1
                continue
            preempted_self = False
            while not self.cache.grow(req.request_id, req.num_computed_tokens + n):
                victim = order.pop()
                self.running.remove(victim)
                self._preempt(victim)
                plan.preempted.append(victim)
                if victim is req:
                    preempted_self = True
                    break
            if preempted_self:
                break
            plan.scheduled.append(ScheduledRequest(req, n))
            budget -= n
            i += 1

        # 2) admissions, unless this step had to preempt
        while not plan.preempted and self.waiting and budget > 0 and len(self.running) < self.max_num_seqs:
            req = self.waiting[0]
            n = min(req.num_tokens - req.num_computed_tokens, budget)
            self.cache.begin(req.request_id)
            if not self.cache.grow(req.request_id, n):
                self.cache.end(req.request_id)
                break
            self.waiting.popleft()
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            plan.scheduled.append(ScheduledRequest(req, n))
            budget -= n
        return plan

    # ------------------------------------------------------------------ update
    def update_from_output(self, plan: StepPlan, sampled: dict) -> list:
        """Apply one step's results: ``sampled`` maps request id -> new token for the requests
        whose portion reached their newest token.  Returns those requests."""
        now = time.monotonic()
        updated = []
        for s in plan.scheduled:
            req = s.request
            req.new_token_ids = []
            req.num_computed_tokens += s.num_tokens
            self.cache.commit(req.request_id, s.num_tokens)
            token = sampled.get(req.request_id)
            if token is None:  # a portion in the middle of the prompt: no logits this step
                continue
            if req.first_token_time is None:
                req.first_token_time = now
            self._append_token(req, int(token))
            updated.append(req)
            if req.finished:
                self.running.remove(req)
                self._release(req)
                req.finish_time = now
        return updated

    # ------------------------------------------------------------------ overlap scheduling
    def _awaiting_last_token(self, req: Request) -> bool:
        """The token it has in flight is the last one it may produce (scheduler.py:417-421)."""
        return req.has_pending_token and (req.num_output_tokens >= req.sampling_params.max_tokens
                                          or req.num_tokens >= self.max_model_len)

    def may_preempt(self) -> bool:
        """Could the next ``schedule`` run out of pages for a running request?  Every running
        request may need one more page, and prompt portions at most a budget's worth."""
        ps = self.cache.page_size
        need = len(self.running) + -(-self.max_num_batched_tokens // ps) + 1
        return any(self.cache.free_pages(g) < need for g in range(len(self.cache.groups)))

    def on_launch(self, plan: StepPlan) -> None:
        """Book a step that has been launched: its tokens count as computed, and every request
        that reaches its newest token gets a placeholder for the token on its way."""
        for s in plan.scheduled:
            req = s.request
            produces = req.num_computed_tokens + s.num_tokens >= req.num_tokens
            req.num_computed_tokens += s.num_tokens
            self.cache.commit(req.request_id, s.num_tokens)
            if produces:
                req.output_token_ids.append(PLACEHOLDER)

    def update_resolved(self, plan: StepPlan, sampled: dict) -> list:
        """The tokens of a launched step have arrived: fill the placeholders in, finish what ends."""
        now = time.monotonic()
        updated = []
        for s in plan.scheduled:
            req = s.request
            token = sampled.get(req.request_id)
            if token is None:
                continue
            req.new_token_ids = []
            if req.finished:  # ended (or was aborted) while this step was in flight: its token is dropped
                del req.output_token_ids[req.num_resolved_outputs:]
                continue
            token = int(token)
            req.output_token_ids[req.num_resolved_outputs] = token
            req.num_resolved_outputs += 1
            req.new_token_ids.append(token)
            if req.first_token_time is None:
                req.first_token_time = now
            updated.append(req)
            if token in req.eos_token_ids or token in req.stop_token_ids:
                status = RequestStatus.FINISHED_STOPPED
            elif (req.num_resolved_outputs >= req.sampling_params.max_tokens
                  or req.num_prompt_tokens + req.num_resolved_outputs >= self.max_model_len):
                status = RequestStatus.FINISHED_LENGTH
            else:
                continue
            del req.output_token_ids[req.num_resolved_outputs:]  # the next step's token, if launched, is dropped
            req.num_computed_tokens = min(req.num_computed_tokens, req.num_tokens)
            if req in self.running:
                self.running.remove(req)
            self._release(req)
            req.status = status
            req.finish_time = now
        return updated

    def _append_token(self, req: Request, token: int) -> None:
        req.output_token_ids.append(token)
        req.num_resolved_outputs = len(req.output_token_ids)
        req.new_token_ids.append(token)
        if token in req.eos_token_ids or token in req.stop_token_ids:
            req.status = RequestStatus.FINISHED_STOPPED
        elif req.num_output_tokens >= req.sampling_params.max_tokens or req.num_tokens >= self.max_model_len:
            req.status = RequestStatus.FINISHED_LENGTH
