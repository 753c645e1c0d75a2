"""What a request may ask of the sampler and of the stopping rules.

The option names and their defaults are 12vivi/tandem's (python/tandem/sampling_params.py:8-19),
so that code written against it carries over.  ``stop`` strings end a request when the decoded
output contains one of them (the text is cut in front of it); they need a tokenizer, and the
engine refuses them at ``add_request`` when it has none.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Union

GREEDY_BELOW = 1e-5  # a temperature under this means argmax (python/tandem/layers/sampler.py:19-21)

# option -> (test of a valid value, the rule in words)
_RULES = {
    "max_tokens": (lambda v: v >= 1, "a request produces at least one token"),
    "temperature": (lambda v: v >= 0, "zero (greedy) or positive"),
    "top_p": (lambda v: 0 < v <= 1, "a probability mass above 0 and up to 1 (1 switches it off)"),
    "min_p": (lambda v: 0 <= v <= 1, "a fraction of the largest probability, 0 to 1 (0 switches it off)"),
}


@dataclass
class SamplingParams:
    max_tokens: int = 16
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1  # zero or less: every token is a candidate
    min_p: float = 0.0
    seed: Optional[int] = None
    stop: Union[str, list, None] = field(default_factory=list)
    stop_token_ids: list = field(default_factory=list)
    ignore_eos: bool = False
    skip_special_tokens: bool = True

    def __post_init__(self) -> None:
        for option, (valid, rule) in _RULES.items():
            value = getattr(self, option)
            if not valid(value):
                raise ValueError(f"SamplingParams.{option} = {value!r} is not allowed: {rule}")
        texts = [self.stop] if isinstance(self.stop, str) else list(self.stop or ())
        if any(not isinstance(t, str) or not t for t in texts):
            raise ValueError(f"SamplingParams.stop takes non-empty strings, got {self.stop!r}")
        self.stop = texts
        self.stop_token_ids = [int(t) for t in (self.stop_token_ids or ())]

    @property
    def greedy(self) -> bool:
        return self.temperature < GREEDY_BELOW
