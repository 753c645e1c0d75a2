"""Continuous batching with chunked prefill under a token budget.

What a step is made of (the rules of 12vivi/tandem's scheduler, python/tandem/scheduler/scheduler.py:216-288,
without its prefix cache, host tier and short-prefill lane):

* requests wait in arrival order and run until they end; a step has ``max_num_batched_tokens``
  tokens to give, and every request it serves takes ``min(tokens it lacks, tokens left)``: a
  prompt is cut wherever the budget ends, and a decoding request lacks exactly one token;
* ``decode_first`` serves the decoding requests, then the requests still reading their prompts,
  then admits from the queue, all in one step; ``prefill_first`` leaves the decoding requests out
  of a step while any prompt work is there, unless that step would come out empty;
* admission stops at the first request that does not fit (budget, ``max_num_seqs``, pages):
  nothing overtakes the head of the queue.

When the pool cannot give a served request its pages, requests are taken from the *end* of the
step's service order (the youngest, not yet served), one at a time, until the pages are there:
each gives back all it holds, forgets how far it had been computed, and moves to the *front* of
the queue, to be read again later with the tokens it has generated.  The request in need may turn
out to be the last one itself.  A step that took pages away admits nobody.  No request may grow
beyond one group's whole pool (``token_capacity``), so the oldest request can always finish and
the queue always drains.

A step's outcome is applied in two halves, because the engine may launch step N before the host
has seen the tokens of step N-1 (overlap scheduling; scheduler.py:409-469 of the reference):
``book_launch`` counts the step's tokens as computed and puts a placeholder where each new token
will go; ``deliver_tokens`` puts the values in, one step later, and ends what has to end.  A
request that ended meanwhile (its token was an end token, or it was aborted) may sit in the step
launched after: that step's token for it is dropped.  A request whose token in flight is the last
it may produce is not served again.  ``update_from_output`` is both halves at once, for a loop
that reads every step's tokens before it plans the next.
"""

from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Optional

from tandem_b200.cache.manager import CacheManager
from tandem_b200.engine.request import Request, RequestStatus

POLICIES = ("prefill_first", "decode_first")


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
        if policy not in POLICIES:
            raise ValueError(f"unknown scheduling policy {policy!r} (known: {', '.join(POLICIES)})")
        self.policy, self.cache = policy, cache
        self.max_num_seqs, self.max_num_batched_tokens = max_num_seqs, max_num_batched_tokens
        self.token_capacity = cache.num_pages * cache.page_size  # what one request can hold when it has the pool to itself
        self.max_model_len = min(max_model_len, self.token_capacity)
        self.waiting: deque = deque()
        self.running: list = []
        self.num_preemptions = 0

    # ------------------------------------------------------------------ requests come and go
    def add_request(self, req: Request) -> None:
        if req.num_prompt_tokens >= self.max_model_len:
            raise ValueError(f"a prompt of {req.num_prompt_tokens} tokens leaves no room for a new token: requests hold at "
                             f"most {self.max_model_len} tokens (max_model_len, and the cache pool of {self.token_capacity})")
        req.status = RequestStatus.WAITING
        self.waiting.append(req)

    def has_unfinished(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    def finish_request(self, req: Request, status: RequestStatus) -> None:
        """End a request from outside the step loop (an abort, a stop string)."""
        if not req.finished:
            self._retire(req, status, time.monotonic())

    def _retire(self, req: Request, status: RequestStatus, now: float) -> None:
        for line in (self.running, self.waiting):
            if req in line:
                line.remove(req)
        self._give_back(req)
        req.drop_unknown()
        req.status, req.finish_time = status, now

    def _give_back(self, req: Request) -> None:
        if self.cache.has(req.request_id):
            self.cache.end(req.request_id)

    # ------------------------------------------------------------------ planning a step
    def schedule(self) -> StepPlan:
        plan = StepPlan()
        prompt_work = bool(self.waiting) or any(not r.is_decoding for r in self.running)
        if self.policy == "prefill_first" and prompt_work:
            self._fill(plan, with_decoding=False)
            if plan.scheduled:
                return plan
        # the same plan goes on: what a first attempt took away stays recorded, and keeps the queue closed
        self._fill(plan, with_decoding=True)
        return plan

    def _service_order(self, with_decoding: bool) -> list:
        reading = [r for r in self.running if not r.is_decoding]
        if not with_decoding:
            return reading
        return [r for r in self.running if r.is_decoding and not self._last_token_in_flight(r)] + reading

    def _fill(self, plan: StepPlan, with_decoding: bool) -> None:
        left = self.max_num_batched_tokens
        line = self._service_order(with_decoding)
        served = 0
        while served < len(line) and left > 0:
            req = line[served]
            share = min(req.tokens_lacking, left)
            if share > 0:
                if not self._make_room(req, share, line, plan):
                    break  # the request itself had to go: nobody is left behind it
                plan.scheduled.append(ScheduledRequest(req, share))
                left -= share
            served += 1
        if not plan.preempted:
            self._admit(plan, left)

    def _make_room(self, req: Request, share: int, line: list, plan: StepPlan) -> bool:
        """Pages for ``share`` more tokens of ``req``, taken from the end of the line if need be.
        False: ``req`` was the end of the line and has been preempted itself."""
        while not self.cache.grow(req.request_id, req.num_computed_tokens + share):
            youngest = line.pop()
            self._preempt(youngest)
            plan.preempted.append(youngest)
            if youngest is req:
                return False
        return True

    def _preempt(self, req: Request) -> None:
        if req.has_pending_token:  # its token would arrive for a request that has started over
            raise RuntimeError(f"request {req.request_id!r} would be preempted with a token in flight "
                               "(the engine reads the step in flight first when may_preempt() says so)")
        self.running.remove(req)
        self._give_back(req)
        req.num_computed_tokens = 0
        req.status = RequestStatus.WAITING
        req.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(req)

    def _admit(self, plan: StepPlan, left: int) -> None:
        while self.waiting and left > 0 and len(self.running) < self.max_num_seqs:
            req = self.waiting[0]
            share = min(req.tokens_lacking, left)
            self.cache.begin(req.request_id)
            if not self.cache.grow(req.request_id, share):
                self.cache.end(req.request_id)
                return  # the head of the queue waits, and so does everyone behind it
            self.waiting.popleft()
            req.status = RequestStatus.RUNNING
            self.running.append(req)
            plan.scheduled.append(ScheduledRequest(req, share))
            left -= share

    def _last_token_in_flight(self, req: Request) -> bool:
        """The token on its way is the last this request may produce."""
        return req.has_pending_token and self._length_reached(req, req.num_output_tokens, req.num_tokens)

    def may_preempt(self) -> bool:
        """Could the next ``schedule`` run short of pages for a running request?  Only running
        requests are ever given pages at another's cost (admission waits instead), so what is
        counted is what they can ask for: each the pages for its lacking tokens, a budget's worth at
        most, beyond the pages it holds, group by group.  The engine then reads the step in flight
        first, so that no request with a placeholder is ever preempted.  A pool that is nearly full of
        decoding requests, the steady state under load, says no here except on the steps in which
        some request begins a page that the pool no longer has."""
        want = [0] * len(self.cache.groups)
        for req in self.running:
            share = min(req.tokens_lacking, self.max_num_batched_tokens)
            if share > 0:
                for g, n in enumerate(self.cache.pages_to_grow(req.request_id, req.num_computed_tokens + share)):
                    want[g] += max(0, n)
        return any(n > self.cache.free_pages(g) for g, n in enumerate(want))

    # ------------------------------------------------------------------ a step's outcome
    def book_launch(self, plan: StepPlan) -> None:
        """The plan's step has been launched: its tokens count as computed, and a request whose
        portion reaches its newest token expects one more."""
        for s in plan.scheduled:
            req = s.request
            req.num_computed_tokens += s.num_tokens
            self.cache.commit(req.request_id, s.num_tokens)
            if req.num_computed_tokens >= req.num_tokens:
                req.expect_token()

    def deliver_tokens(self, plan: StepPlan, sampled: dict) -> list:
        """The tokens of a launched step have arrived (request id -> token, for the requests that
        were promised one).  Returns the requests that got a token, ended ones included."""
        now = time.monotonic()
        got = []
        for s in plan.scheduled:
            req = s.request
            if req.request_id not in sampled:
                continue  # a portion inside the prompt
            req.new_token_ids = []
            if req.finished:
                continue  # ended while this step was in flight: its token is of no use
            token = int(sampled[req.request_id])
            req.receive_token(token)
            if req.first_token_time is None:
                req.first_token_time = now
            got.append(req)
            ended = self._ending(req, token)
            if ended is not None:
                self._retire(req, ended, now)
        return got

    def update_from_output(self, plan: StepPlan, sampled: dict) -> list:
        """Both halves at once: for a loop that reads each step's tokens before planning the next."""
        for s in plan.scheduled:
            s.request.new_token_ids = []
        self.book_launch(plan)
        return self.deliver_tokens(plan, sampled)

    def _length_reached(self, req: Request, outputs: int, tokens: int) -> bool:
        return outputs >= req.sampling_params.max_tokens or tokens >= self.max_model_len

    def _ending(self, req: Request, token: int) -> Optional[RequestStatus]:
        if token in req.end_tokens:
            return RequestStatus.FINISHED_STOPPED
        if self._length_reached(req, req.num_known_outputs, req.num_known):
            return RequestStatus.FINISHED_LENGTH
        return None
