"""Rotary position encoding: the angle table.

inv_freq[j] = theta^(-2j / rotary_dim), angle = position * inv_freq, all float32 and built on
the host exactly as 12vivi/tandem builds them (python/tandem/layers/rotary.py:10-13,41-49).  The table
is [max_position, rotary_dim] = [cos of the rotary_dim/2 angles | sin of them]
(the ``cos_sin_cache`` layout of rotary.py:49); the attention mixer's prologue kernel applies it
with the rotate_half pairing (j, j + rotary_dim/2).
"""

from __future__ import annotations

import torch

from tandem_b200.config.plan import PositionSpec


class RotaryTable:
    def __init__(self, spec: PositionSpec, device) -> None:
        if spec.rotary_dim <= 0 or spec.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be positive and even, got {spec.rotary_dim}")
        self.rotary_dim = spec.rotary_dim
        inv_freq = 1.0 / (spec.theta ** (torch.arange(0, spec.rotary_dim, 2, dtype=torch.int64).to(torch.float32)
                                         / spec.rotary_dim))
        freqs = torch.outer(torch.arange(spec.max_position, dtype=torch.float32), inv_freq)
        self.cos_sin = torch.cat([freqs.cos(), freqs.sin()], dim=-1).contiguous().to(device)


class NoPosition:
    """kind "none": tokens carry no position encoding."""

    rotary_dim = 0
    cos_sin = None

    def __init__(self, spec: PositionSpec, device) -> None:
        pass
