"""One generation request, as the scheduler and the engine see it, and what the caller gets back.

A request is one list of tokens: its prompt, then what it has generated.  Three counters run
along that list:

* ``num_computed_tokens``: tokens whose cache entries are stored (or on their way in a launched
  step).  Every step hands the request tokens until this has caught up with the list, so a
  prompt portion and a decoded token are the same operation, and a request that lost its pages
  is simply read again from the start, generated tokens included
  (python/tandem/engine/request.py:125-127 of 12vivi/tandem keeps the same count);
* ``num_known``: leading tokens whose values the host knows.  With overlap scheduling the newest
  token may still be on the device; its place in the list holds ``PLACEHOLDER`` until it arrives;
* the length of the list itself.
"""

from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field
from typing import Optional, Sequence

from tandem_b200.sampling.params import SamplingParams

PLACEHOLDER = -1  # stands in the token list for a token that a launched step will produce


class RequestStatus(enum.Enum):
    """Where a request is; the value of an ended status is the ``finish_reason`` callers see."""

    WAITING = "waiting"
    RUNNING = "running"
    FINISHED_STOPPED = "stop"  # an end token, a stop token or a stop string
    FINISHED_LENGTH = "length"  # max_tokens or the model's length
    FINISHED_ABORTED = "abort"

    @property
    def finished(self) -> bool:
        return self.name.startswith("FINISHED")


class Request:
    def __init__(self, request_id: str, prompt_token_ids: Sequence[int], sampling_params: SamplingParams,
                 eos_token_ids: Sequence[int] = (), sample_seed: int = 0, arrival_time: Optional[float] = None) -> None:
        self.request_id = request_id
        self.sampling_params = sampling_params
        self.token_ids = [int(t) for t in prompt_token_ids]
        self.num_prompt_tokens = len(self.token_ids)
        self.num_known = self.num_prompt_tokens
        self.num_computed_tokens = 0
        # a generated token from this set ends the request (the model's end tokens unless ignored)
        self.end_tokens = frozenset(sampling_params.stop_token_ids) | \
            (frozenset() if sampling_params.ignore_eos else frozenset(int(t) for t in eos_token_ids))
        self.status = RequestStatus.WAITING
        self.sample_seed = sample_seed  # the k-th generated token is drawn with uniform(sample_seed, k)
        self.inflight_row = -1  # row of the launched step's token tensor that holds the placeholder's value
        self.new_token_ids: list = []  # tokens that arrived with the latest step
        self.num_preemptions = 0
        self.arrival_time = time.monotonic() if arrival_time is None else arrival_time
        self.first_token_time: Optional[float] = None
        self.finish_time: Optional[float] = None
        self.text = None  # engine.text.OutputText when the engine has a tokenizer

    # ------------------------------------------------------------------ the token list
    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def prompt_token_ids(self) -> list:
        return self.token_ids[: self.num_prompt_tokens]

    @property
    def output_token_ids(self) -> list:
        """Generated tokens whose values are known (none in flight)."""
        return self.token_ids[self.num_prompt_tokens: self.num_known]

    @property
    def num_output_tokens(self) -> int:
        """Generated tokens, the one in flight included."""
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def num_known_outputs(self) -> int:
        return self.num_known - self.num_prompt_tokens

    @property
    def has_pending_token(self) -> bool:
        return self.num_known < len(self.token_ids)

    @property
    def tokens_lacking(self) -> int:
        """Tokens that still have to go through the model before the next one can be sampled."""
        return len(self.token_ids) - self.num_computed_tokens

    @property
    def is_decoding(self) -> bool:
        """All but the newest token are stored, and that newest token was generated."""
        return self.tokens_lacking == 1 and len(self.token_ids) > self.num_prompt_tokens

    def next_tokens(self, n: int) -> list:
        return self.token_ids[self.num_computed_tokens: self.num_computed_tokens + n]

    # ------------------------------------------------------------------ generated tokens
    def expect_token(self) -> None:
        """A launched step will produce this request's next token."""
        self.token_ids.append(PLACEHOLDER)

    def receive_token(self, token: int) -> None:
        """The value of the oldest token in flight has arrived (or, with nothing in flight, a
        token that was sampled and read in the same step)."""
        if self.num_known == len(self.token_ids):
            self.token_ids.append(token)
        else:
            self.token_ids[self.num_known] = token
        self.num_known += 1
        self.new_token_ids.append(token)

    def drop_unknown(self) -> None:
        """Forget tokens still in flight (the request has ended: they will not be used)."""
        del self.token_ids[self.num_known:]
        self.num_computed_tokens = min(self.num_computed_tokens, len(self.token_ids))

    # ------------------------------------------------------------------ status
    @property
    def finished(self) -> bool:
        return self.status.finished

    @property
    def finish_reason(self) -> Optional[str]:
        return self.status.value if self.status.finished else None

    def __repr__(self) -> str:  # pragma: no cover
        return (f"<Request {self.request_id} {self.status.name}: {self.num_prompt_tokens} prompt + "
                f"{self.num_output_tokens} generated, {self.num_computed_tokens} computed>")


@dataclass
class RequestOutput:
    request_id: str
    prompt_token_ids: list
    output_token_ids: list  # all generated tokens once the request has finished, empty before
    text: str
    delta_token_ids: list
    finished: bool
    finish_reason: Optional[str]
    metrics: dict = field(default_factory=dict)
    num_output_tokens: int = 0
    delta_text: str = ""
