"""Counter-based uniform numbers for sampling.

The k-th token of a request is drawn with ``uniform(seed, k)``: a pure function, so a draw
depends neither on the other requests of the batch nor on how the request was cut into steps,
and a preempted request that is recomputed draws the same tokens again.  12vivi/tandem keeps a
``torch.Generator`` per seeded request instead (python/tandem/engine/llm_engine.py:263-264).
"""

from __future__ import annotations

_MASK = (1 << 64) - 1


def _mix(x: int) -> int:
    """splitmix64 finaliser."""
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform(seed: int, counter: int) -> float:
    """A number in [0, 1) with 24 random bits (exact in float32)."""
    return (_mix(_mix(seed & _MASK) ^ (counter & _MASK)) >> 40) / float(1 << 24)
