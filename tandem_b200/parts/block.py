"""Arrangements of a layer's parts around the residual stream.

"prenorm": h <- h + mixer(norm(h)); h <- h + feed_forward(norm(h)), carried as the pair
(x = the last sublayer's output, residual = the float32 stream) so that every "add, then
normalise" is one kernel (12vivi/tandem python/tandem/models/llama_family.py:11-16,59-67).
"""

from __future__ import annotations

from typing import Optional

import torch

from tandem_b200.kernels import ops
from tandem_b200.parts.base import StepContext


def norm_input(norm, x):
    """What a mixer or a feed-forward returned, as the norm behind it can take it: the matrix
    products of this package may return a split output, which norms that declare
    ``takes_split_input`` add up themselves and all others get as a tensor."""
    return x if getattr(norm, "takes_split_input", False) else ops.as_tensor(x)


class PreNormBlock:
    def forward(self, layer, x, residual: torch.Tensor, ctx: StepContext):
        h = layer.mixer_norm.forward(norm_input(layer.mixer_norm, x), residual, ctx.dtype)
        a = layer.mixer.forward(h, ctx)
        h = layer.feed_forward_norm.forward(norm_input(layer.feed_forward_norm, a), residual, ctx.dtype)
        return layer.feed_forward.forward(h, ctx)
