"""One generation request and what comes back from it
(python/tandem/engine/request.py:18-155, without the prefix-cache and speculative fields)."""

from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Optional

from tandem_b200.sampling.params import SamplingParams


PLACEHOLDER = -1  # an output token that a launched step will produce and the host has not seen yet


class RequestStatus(enum.Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED_STOPPED = "stop"
    FINISHED_LENGTH = "length"
    FINISHED_ABORTED = "abort"

    @property
    def finished(self) -> bool:
        return self in (RequestStatus.FINISHED_STOPPED, RequestStatus.FINISHED_LENGTH, RequestStatus.FINISHED_ABORTED)


class Request:
    """Bookkeeping in "computed tokens": ``num_computed_tokens`` counts tokens whose cache
    entries are stored; every step hands the request tokens until it has caught up with
    ``num_tokens``.  A prompt portion and a decoded token are the same operation."""

    def __init__(self, request_id: str, prompt_token_ids: list, sampling_params: SamplingParams,
                 eos_token_ids=None, sample_seed: int = 0, arrival_time: Optional[float] = None) -> None:
        self.request_id = request_id
        self.prompt_token_ids = list(prompt_token_ids)
        self.sampling_params = sampling_params
        self.eos_token_ids = set() if sampling_params.ignore_eos else set(eos_token_ids or [])
        self.stop_token_ids = set(sampling_params.stop_token_ids)
        self.output_token_ids: list = []
        self.new_token_ids: list = []
        self.status = RequestStatus.WAITING
        self.num_computed_tokens = 0
        self.sample_seed = sample_seed  # the k-th output token is drawn with uniform(sample_seed, k)
        self.arrival_time = time.monotonic() if arrival_time is None else arrival_time
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None
        self.num_preemptions = 0
        self.num_resolved_outputs = 0  # output tokens whose values the host knows (overlap scheduling)
        self.inflight_row = -1  # row of the launched step's token tensor that holds the placeholder's value

    @property
    def has_pending_token(self) -> bool:
        return self.num_resolved_outputs < len(self.output_token_ids)

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_output_tokens(self) -> int:
        return len(self.output_token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.prompt_token_ids) + len(self.output_token_ids)

    def token_ids_in_range(self, start: int, end: int) -> list:
        p = len(self.prompt_token_ids)
        if start >= p:
            return self.output_token_ids[start - p: end - p]
        if end <= p:
            return self.prompt_token_ids[start:end]
        return self.prompt_token_ids[start:] + self.output_token_ids[: end - p]

    @property
    def is_decoding(self) -> bool:
        return self.num_computed_tokens == self.num_tokens - 1 and self.num_output_tokens > 0

    @property
    def finished(self) -> bool:
        return self.status.finished

    @property
    def finish_reason(self) -> Optional[str]:
        return self.status.value if self.status.finished else None

    def __repr__(self) -> str:  # pragma: no cover
        return (f"Request({self.request_id}, {self.status.name}, prompt={self.num_prompt_tokens}, "
                f"out={self.num_output_tokens}, computed={self.num_computed_tokens})")


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: list
    output_token_ids: list
    text: str
    delta_token_ids: list
    finished: bool
    finish_reason: Optional[str]
    metrics: dict = field(default_factory=dict)
    num_output_tokens: int = 0
