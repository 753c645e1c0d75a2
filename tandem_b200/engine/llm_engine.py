"""The engine a user holds: requests in, tokens out.

``LLMEngine`` wires configuration, model, cache manager, scheduler, step function and sampler
(12vivi/tandem python/tandem/engine/llm_engine.py:38-175), with the same calls: ``add_request``,
``step``, ``generate``, ``abort_request``, ``stats``.  Prompts are lists of token ids; text
prompts need a tokenizer, which this engine loads only when the model folder has one.
``LLM`` is the short spelling: ``LLM(model=...).generate(prompts, sampling_params)``.
"""

from __future__ import annotations

import itertools
import os
import time
from typing import Optional, Sequence, Union

import torch

from tandem_b200.config.engine_config import EngineConfig
from tandem_b200.engine.core import build_executor, load_model
from tandem_b200.engine.executor import StepEntry
from tandem_b200.engine.request import PLACEHOLDER, Request, RequestOutput, RequestStatus
from tandem_b200.engine.scheduler import Scheduler, StepPlan
from tandem_b200.engine.text import OutputText
from tandem_b200.kernels import ops
from tandem_b200.sampling.params import SamplingParams
from tandem_b200.sampling.sampler import sample_on_device

PromptType = Union[str, Sequence[int]]


class _InFlight:
    """A launched step: its plan, the requests that get a token from it (in the order of the
    rows of ``tokens``), the tokens on the device, and their copy to pinned host memory with the
    event that says it has landed."""

    def __init__(self, plan: StepPlan, requests: list, tokens: torch.Tensor) -> None:
        self.plan, self.requests, self.tokens = plan, requests, tokens
        self.host = None
        self.event = None
        if tokens.is_cuda:
            # the tokens and, behind them, the word in which kernels record a fault they survived
            n = tokens.numel()
            self.host = torch.empty(n + 1, dtype=torch.int32, pin_memory=True)
            self.host[:n].copy_(tokens, non_blocking=True)
            self.host[n:].copy_(ops.status_word(tokens.device), non_blocking=True)
            self.event = torch.cuda.Event()
            self.event.record()

    def resolve(self) -> dict:
        """Request id -> token.  Raises ``KernelError`` if a kernel of the step recorded a fault (a
        bounded wait that gave up, a missing page): its tokens were sampled from invalid logits."""
        if self.event is not None:
            self.event.synchronize()
            values = self.host.tolist()
            status = values.pop()
            if status:
                ops.raise_status(self.tokens.device, status)
        else:
            values = self.tokens.tolist()
        return {r.request_id: t for r, t in zip(self.requests, values)}


class LLMEngine:
    def __init__(self, config: EngineConfig, decoder=None, model_config=None, tokenizer=None,
                 load_tokenizer: bool = True) -> None:
        """``decoder`` / ``model_config``: a model that is already built (random weights made on
        the device, tests); otherwise ``config.model`` is a folder read through the registry."""
        self.config = config
        if decoder is None:
            decoder, model_config = load_model(config.model, config.resolved_dtype, config.device)
        self.decoder, self.model_config = decoder, model_config
        plan = decoder.plan
        self.max_model_len = config.max_model_len or min(plan.max_position, 32768)  # llm_engine.py:55
        if self.max_model_len > plan.max_position:
            raise ValueError(f"max_model_len {self.max_model_len} exceeds the model's {plan.max_position} positions")
        self.executor = build_executor(decoder, config.block_size, config.num_kv_blocks, config.kv_cache_memory_gb,
                                       config.max_num_seqs)
        self.cache = self.executor.manager
        self.scheduler = Scheduler(self.cache, config.max_num_seqs, config.max_num_batched_tokens,
                                   self.max_model_len, config.schedule_policy)
        self.eos_token_ids = list(plan.eos_token_ids)
        self.tokenizer = tokenizer
        if tokenizer is None and load_tokenizer and config.model and \
                os.path.isfile(os.path.join(config.model, "tokenizer.json")):
            from transformers import AutoTokenizer  # text in and out only; no model code

            self.tokenizer = AutoTokenizer.from_pretrained(config.model)
        # Overlap scheduling (llm_engine.py:298-346 of the reference): step N is launched before the
        # host has seen the tokens of step N-1, which enter N's batch on the device.
        self.overlap = bool(config.overlap_schedule)
        self.inflight: Optional[_InFlight] = None
        self.requests: dict = {}
        self._ids = itertools.count()
        self.num_steps = 0
        self.trace = None  # engine.trace.TraceWriter: every launched step, in the replay tool's format
        if not config.small_batch_gemv:
            from tandem_b200.kernels import gemm_bf16

            gemm_bf16.keep_library_products()
        self.graphs = None
        if config.cuda_graph:
            from tandem_b200.engine.cuda_graph import DecodeGraphs

            self.graphs = DecodeGraphs.maybe(self.executor, config.cuda_graph_max_bs, self.max_model_len)
            if self.graphs is not None and config.cuda_graph_capture_at_start:
                self.graphs.capture_all()

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: Optional[PromptType] = None, sampling_params: Optional[SamplingParams] = None,
                    request_id: Optional[str] = None, prompt_token_ids: Optional[Sequence[int]] = None) -> str:
        sp = sampling_params or SamplingParams()
        if prompt_token_ids is None:
            if isinstance(prompt, str):
                if self.tokenizer is None:
                    raise ValueError("text prompts need a tokenizer; pass token ids")
                prompt_token_ids = self.tokenizer.encode(prompt)
            elif prompt is not None:
                prompt_token_ids = list(prompt)
            else:
                raise ValueError("either prompt or prompt_token_ids is required")
        if not prompt_token_ids:
            raise ValueError("empty prompt")
        vocab = self.decoder.plan.embedding.vocab_size
        for t in prompt_token_ids:
            if not 0 <= int(t) < vocab:
                raise ValueError(f"token id {t} is outside the vocabulary [0, {vocab})")
        if len(prompt_token_ids) >= self.max_model_len:
            raise ValueError(f"prompt has {len(prompt_token_ids)} tokens; max_model_len is {self.max_model_len}")
        if sp.stop and self.tokenizer is None:
            raise ValueError("stop strings are matched against decoded text and need a tokenizer; this engine has none "
                             "(use stop_token_ids, or give the engine a tokenizer)")
        index = next(self._ids)
        rid = request_id or f"req-{index}"
        if rid in self.requests:
            raise ValueError(f"duplicate request id {rid}")
        # a request without a seed draws from the engine's seed and its own arrival number
        seed = sp.seed if sp.seed is not None else (self.config.seed * 1_000_003 + index + 1)
        req = Request(rid, list(prompt_token_ids), sp, self.eos_token_ids, sample_seed=seed)
        if self.tokenizer is not None:
            req.text = OutputText(self.tokenizer, sp.skip_special_tokens, sp.stop)
        self.scheduler.add_request(req)
        self.requests[rid] = req
        return rid

    def abort_request(self, request_id: str) -> None:
        req = self.requests.pop(request_id, None)
        if req is not None and not req.finished:
            self.scheduler.finish_request(req, RequestStatus.FINISHED_ABORTED)

    def has_unfinished_requests(self) -> bool:
        return self.scheduler.has_unfinished() or self.inflight is not None

    # ------------------------------------------------------------------ step
    def step(self) -> list:
        """schedule -> run -> sample -> update (llm_engine.py:284-296 of 12vivi/tandem).  With
        overlap scheduling a call launches one step and returns the outputs of the step launched
        by the call before, whose tokens the host reads while the new step runs."""
        if self.overlap:
            return self._step_overlap()
        plan = self.scheduler.schedule()
        if plan.is_empty:
            if self.scheduler.has_unfinished() and not plan.preempted:
                raise RuntimeError("the scheduler could place no request: the cache pool is too small")
            return []
        launched = self._launch(plan)
        updated = self.scheduler.update_from_output(plan, launched.resolve())
        self.num_steps += 1
        return self._emit(updated)

    def _step_overlap(self) -> list:
        outputs = []
        if self.inflight is not None and self.scheduler.may_preempt():
            outputs = self.drain()  # pages are short: no request with a token in flight may be preempted
        plan = self.scheduler.schedule()
        launched = None
        if not plan.is_empty:
            launched = self._launch(plan)
            self.scheduler.book_launch(plan)
            for row, req in enumerate(launched.requests):
                req.inflight_row = row
            self.num_steps += 1
        elif self.inflight is None and not outputs and self.scheduler.has_unfinished() and not plan.preempted:
            raise RuntimeError("the scheduler could place no request: the cache pool is too small")
        previous, self.inflight = self.inflight, launched
        self.executor.pending_tokens = launched.tokens if launched is not None else None
        if previous is not None:
            outputs += self._emit(self.scheduler.deliver_tokens(previous.plan, previous.resolve()))
        return outputs

    def drain(self) -> list:
        """Wait for the step in flight, if any, and apply its tokens."""
        previous, self.inflight = self.inflight, None
        self.executor.pending_tokens = None
        if previous is None:
            return []
        return self._emit(self.scheduler.deliver_tokens(previous.plan, previous.resolve()))

    def _emit(self, updated: list) -> list:
        outputs = []
        for req in updated:
            delta = ""
            if req.text is not None:
                delta = req.text.feed(req.output_token_ids, req.finished)
                if req.text.stopped and not req.finished:  # llm_engine.py:382-383 of the reference
                    self.scheduler.finish_request(req, RequestStatus.FINISHED_STOPPED)
            outputs.append(self._make_output(req, delta))
            if req.finished:
                self.requests.pop(req.request_id, None)
        return outputs

    def entries_of(self, plan: StepPlan) -> list:
        """The plan as step entries: logits are wanted only at the last token of a portion that
        reaches the request's newest token (python/tandem/executor/model_runner.py:102-105)."""
        entries = []
        for s in plan.scheduled:
            req, n = s.request, s.num_tokens
            tokens = req.next_tokens(n)
            # only the newest token can still be on its way (model_runner.py:95-99 of the reference)
            pending = req.inflight_row if tokens[-1] == PLACEHOLDER else None
            reaches_newest = req.num_computed_tokens + n >= req.num_tokens
            entries.append(StepEntry(req.request_id, tokens, [n - 1] if reaches_newest else [], pending))
        return entries

    def record_steps(self, path: str) -> None:
        """Write every step from now on to ``path`` as the replay tool reads it (one JSON object a
        line), so that this run's logits can be reproduced and dumped by ``trace_run``.  What
        12vivi/tandem's TANDEM_TRACE records of a step (python/tandem/executor/step_timer.py:57-68),
        with the tokens themselves added."""
        from tandem_b200.engine.trace import TraceWriter

        self.drain()
        self.trace = TraceWriter(path)

    def _launch(self, plan: StepPlan) -> _InFlight:
        """Run the plan's step and its sampling on the device; nothing is read back here."""
        entries = self.entries_of(plan)
        if self.trace is not None:
            self.trace.step(plan, entries)
        sampling = [s.request for s, e in zip(plan.scheduled, entries) if e.want]
        if self.graphs is not None and self.graphs.takes(entries):
            logits = self.graphs.run(entries)
        else:
            logits = self.executor.run(entries)
        if sampling:
            tokens = sample_on_device(logits, [r.sampling_params for r in sampling], [r.sample_seed for r in sampling],
                                      [r.num_output_tokens for r in sampling])
        else:
            tokens = torch.empty(0, dtype=torch.int32, device=logits.device)
        return _InFlight(plan, sampling, tokens)

    def _make_output(self, req: Request, delta_text: str = "") -> RequestOutput:
        metrics = {}
        if req.first_token_time is not None:
            metrics["ttft"] = req.first_token_time - req.arrival_time
        if req.finished and req.finish_time is not None:
            metrics["latency"] = req.finish_time - req.arrival_time
            metrics["preemptions"] = req.num_preemptions
        text = req.text.text if req.text is not None else ""
        return RequestOutput(req.request_id, req.prompt_token_ids, req.output_token_ids if req.finished else [], text,
                             list(req.new_token_ids), req.finished, req.finish_reason, metrics, req.num_known_outputs,
                             delta_text)

    # ------------------------------------------------------------------ offline API
    def generate(self, prompts: Sequence[PromptType],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> list:
        """Run the prompts to completion; outputs in the order of the prompts (llm_engine.py:411-426)."""
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            params = [sampling_params or SamplingParams()] * len(prompts)
        else:
            params = list(sampling_params)
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        final = {}
        while self.has_unfinished_requests():
            for out in self.step():
                if out.finished:
                    final[out.request_id] = out
        return [final[i] for i in ids]

    def stats(self) -> dict:
        return {
            "steps": self.num_steps,
            "free_kv_blocks": self.cache.free_pages(0) if self.cache.groups else 0,
            "total_kv_blocks": self.cache.num_pages,
            "running": len(self.scheduler.running),
            "waiting": len(self.scheduler.waiting),
            "preemptions": self.scheduler.num_preemptions,
        }


class LLM:
    """``LLM(model=folder, dtype=..., **engine options).generate(prompts, sampling_params)``."""

    def __init__(self, model: str, **options) -> None:
        self.engine = LLMEngine(EngineConfig(model=model, **options))

    def generate(self, prompts: Sequence[PromptType],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None) -> list:
        return self.engine.generate(prompts, sampling_params)

    def stats(self) -> dict:
        return self.engine.stats()
