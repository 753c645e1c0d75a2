"""Arrangements of a layer's parts around the residual stream.

"prenorm": h <- h + mixer(norm(h)); h <- h + feed_forward(norm(h)), carried as the pair
(x = the last sublayer's output, residual = the float32 stream) so that every "add, then
normalise" is one kernel (12vivi/tandem python/tandem/models/llama_family.py:11-16,59-67).
"""

from __future__ import annotations

from typing import Optional

import torch

from tandem_b200.parts.base import StepContext


class PreNormBlock:
    def forward(self, layer, x: Optional[torch.Tensor], residual: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        h = layer.mixer_norm.forward(x, residual, ctx.dtype)
        a = layer.mixer.forward(h, ctx)
        h = layer.feed_forward_norm.forward(a, residual, ctx.dtype)
        return layer.feed_forward.forward(h, ctx)
