"""Arrangements of a layer's parts around the residual stream.

"prenorm": h <- h + mixer(norm(h)); h <- h + feed_forward(norm(h)), carried as the pair
(x = the last sublayer's output, residual = the float32 stream) so that every "add, then
normalise" is one kernel (12vivi/tandem python/tandem/models/llama_family.py:11-16,59-67).

An arrangement declares the parts it works with as ``slots`` (slot name -> family; all needed)
and ``optional_slots``; the decoder builds what the layer's spec lists under those names and
hands the arrangement a layer whose attributes they are.  ``forward(layer, x, residual, ctx)``
gets the last sublayer's output ``x`` (None in front of the first layer) and the float32
residual stream, and returns its own last sublayer's output, not yet added to the stream.
"""

from __future__ import annotations

from typing import Optional

import torch

from tandem_b200.kernels import ops
from tandem_b200.parts.base import StepContext


class PreNormBlock:
    slots = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}

    def forward(self, layer, x, residual: torch.Tensor, ctx: StepContext):
        h = layer.mixer_norm.forward(x, residual, ctx.dtype)
        a = layer.mixer.forward(h, ctx)
        h = layer.feed_forward_norm.forward(a, residual, ctx.dtype)
        return layer.feed_forward.forward(h, ctx)
