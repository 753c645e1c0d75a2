"""Arrangements of a layer's parts around the residual stream.

"prenorm": h <- h + mixer(norm(h)); h <- h + feed_forward(norm(h)), carried as the pair
(x = the last sublayer's output, residual = the float32 stream) so that every "add, then
normalise" is one kernel (12vivi/tandem python/tandem/models/llama_family.py:11-16,59-67).

An arrangement declares the parts it works with as ``slots`` (slot name -> family; all needed)
and ``optional_slots``; the decoder builds what the layer's spec lists under those names and
hands the arrangement a layer whose attributes they are.  ``forward(layer, x, residual, ctx)``
gets the last sublayer's output ``x`` (None in front of the first layer) and the float32
residual stream, and returns its own last sublayer's output, not yet added to the stream.

Values between parts may be *pending* (``tandem_b200.kernels.deferred``): a product that its
norm will have added into the residual by the product's own kernel, a norm whose rows' scale the
product behind it applies.  Only parts that declare ``takes_deferred = True`` are handed such
values or asked for them (``forward(..., defer=True)``); an arrangement that declares it may get a
pending ``x`` and return one.
"""

from __future__ import annotations

from typing import Optional

import torch

from tandem_b200.kernels import deferred
from tandem_b200.parts.base import StepContext


def lazy(part) -> bool:
    return getattr(part, "takes_deferred", False)


def normed(norm, x, residual: torch.Tensor, ctx: StepContext, reader):
    """``norm`` applied to residual + x for the part ``reader``; pending where both can deal with it."""
    if lazy(norm):
        return norm.forward(x, residual, ctx.dtype, defer=lazy(reader))
    return norm.forward(deferred.tensor(x), residual, ctx.dtype)


def run(part, h, ctx: StepContext):
    """A mixer or feed-forward on ``h``; its last product may come back pending if the part knows how."""
    return part.forward(h, ctx, defer=True) if lazy(part) else part.forward(deferred.tensor(h), ctx)


class PreNormBlock:
    slots = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}
    takes_deferred = True

    def forward(self, layer, x, residual: torch.Tensor, ctx: StepContext):
        h = normed(layer.mixer_norm, x, residual, ctx, layer.mixer)
        a = run(layer.mixer, h, ctx)
        h = normed(layer.feed_forward_norm, a, residual, ctx, layer.feed_forward)
        return run(layer.feed_forward, h, ctx)
