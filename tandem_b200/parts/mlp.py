"""Gated feed-forward (SwiGLU): down(act(gate(x)) * up(x)) with gate and up as one product
(12vivi/tandem python/tandem/layers/mlp.py:23-44; rows [gate | up] as python/tandem/models/loader.py:52-53
stacks them)."""

from __future__ import annotations

import torch

from tandem_b200.config.model_config import ConfigError
from tandem_b200.config.plan import GatedMLPSpec, ParamSpec, WeightSource
from tandem_b200.kernels import ops
from tandem_b200.parts.base import FeedForward, StepContext


class GatedMLP(FeedForward):
    takes_deferred = True  # x may be a norm whose scale is pending; with ``defer`` the last product may stay pending

    @staticmethod
    def params(spec: GatedMLPSpec) -> dict:
        H, I, p = spec.hidden_size, spec.intermediate_size, spec.prefix
        return {
            "gate_up": ParamSpec((2 * I, H), (WeightSource(f"{p}.gate_proj.weight", 0, I),
                                              WeightSource(f"{p}.up_proj.weight", I, I))),
            "down": ParamSpec((H, I), (WeightSource(f"{p}.down_proj.weight"),)),
        }

    def __init__(self, spec: GatedMLPSpec, weights: dict, dtype: torch.dtype, device) -> None:
        if spec.activation != "silu":
            raise ConfigError(f"gated_mlp has no activation {spec.activation!r} (only silu)")
        self.gate_up = weights["gate_up"]
        self.down = weights["down"]

    def forward(self, x, ctx: StepContext, defer: bool = False):
        return ops.linear(ops.gated_linear(x, self.gate_up), self.down, defer=defer)
