"""RMSNorm with the residual add fused in front of it.

y = weight * x * rsqrt(mean(x^2) + eps), all in float32
(12vivi/tandem python/tandem/layers/norm.py:15-19, python/tandem/layers/ops.py:29-42); the
residual stream it adds into is float32 in both modes.
"""

from __future__ import annotations

from typing import Optional

import torch

from tandem_b200.config.plan import NormSpec, ParamSpec, WeightSource
from tandem_b200.kernels import ops
from tandem_b200.parts.base import Norm


class RMSNorm(Norm):
    takes_deferred = True  # x may be a product that is still pending; the result may stay pending (kernels/deferred.py)

    @staticmethod
    def params(spec: NormSpec) -> dict:
        return {"weight": ParamSpec((spec.size,), (WeightSource(spec.weight),), role="vector")}

    def __init__(self, spec: NormSpec, weights: dict, dtype: torch.dtype, device) -> None:
        self.eps = spec.eps
        self.weight = weights["weight"]

    def forward(self, x, residual: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None,
                defer: bool = False):
        return ops.add_rmsnorm(x, residual, self.weight, self.eps, out_dtype, rows, defer=defer)
