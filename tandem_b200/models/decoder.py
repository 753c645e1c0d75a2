"""The generic decoder: embedding, the plan's runs in order, final norm, output head.

It is built from a :class:`~tandem_b200.config.plan.ModelPlan` and a source of checkpoint
tensors, looks every part up by kind in the registry, and knows no architecture by name.  The
loop is the one of 12vivi/tandem's python/tandem/models/llama_family.py:86-116 with the layer
order read from the plan instead of ``range(num_layers)``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional

import torch

from tandem_b200.config.plan import ModelPlan, ParamSpec, WeightSource
from tandem_b200.kernels import ops
from tandem_b200.parts.base import StepContext
from tandem_b200.parts.block import norm_input
from tandem_b200.registry import part
from tandem_b200.weights.loader import TensorSource, load_parameters


@dataclass
class Layer:
    block: Any
    mixer_norm: Any
    mixer: Any
    feed_forward_norm: Any
    feed_forward: Any


_SLOTS = (("mixer_norm", "norm"), ("mixer", "mixer"), ("feed_forward_norm", "norm"), ("feed_forward", "feed_forward"))


class Decoder:
    def __init__(self, plan: ModelPlan, source: TensorSource, dtype: torch.dtype, device) -> None:
        self.plan, self.dtype, self.device = plan, dtype, torch.device(device)
        e, h = plan.embedding, plan.head
        params: dict[str, ParamSpec] = {"embedding": ParamSpec((e.vocab_size, e.hidden_size), (WeightSource(e.weight),))}
        for i, layer in enumerate(plan.layers):
            for slot, family in _SLOTS:
                spec = getattr(layer, slot)
                for local, ps in part(family, spec.kind).params(spec).items():
                    params[f"layers.{i}.{slot}.{local}"] = ps
        for local, ps in part("norm", plan.final_norm.kind).params(plan.final_norm).items():
            params[f"final_norm.{local}"] = ps
        if h.weight is not None:
            params["head"] = ParamSpec((h.vocab_size, h.hidden_size), (WeightSource(h.weight),))
        tensors = load_parameters(params, source, dtype, device, plan.ignored_weights)

        def weights_of(prefix: str) -> dict:
            return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}

        self.embedding = tensors["embedding"]
        self.head = tensors.get("head", self.embedding)  # tied: llama_family.py:108
        self.layers = []
        for i, layer in enumerate(plan.layers):
            built = {}
            for slot, family in _SLOTS:
                spec = getattr(layer, slot)
                built[slot] = part(family, spec.kind)(spec, weights_of(f"layers.{i}.{slot}."), dtype, self.device)
            self.layers.append(Layer(block=part("block", layer.block)(), **built))
        self.final_norm = part("norm", plan.final_norm.kind)(plan.final_norm, weights_of("final_norm."), dtype,
                                                             self.device)
        self.num_parameters = sum(t.numel() for t in tensors.values())
        self.parameter_bytes = sum(t.numel() * t.element_size() for t in tensors.values())

    # what the cache manager has to provide for each run of the plan
    def kv_needs(self) -> list:
        out = []
        for run in self.plan.order:
            spec = self.plan.layers[run.layer].mixer
            out.append(None if run.cache_of is not None else part("mixer", spec.kind).kv_need(spec))
        return out

    def state_needs(self) -> list:
        out = []
        for run in self.plan.order:
            spec = self.plan.layers[run.layer].mixer
            out.append(part("mixer", spec.kind).state_need(spec))
        return out

    def forward(self, ctx: StepContext, logit_rows: Optional[torch.Tensor]) -> torch.Tensor:
        """Logits float32 [R, vocab] at the rows ``logit_rows`` (int32 indices into the step's
        tokens; None: every token).  Runs only the tokens of the step, from the cache."""
        if ctx.num_tokens == 0:
            return torch.empty((0, self.plan.head.vocab_size), dtype=torch.float32, device=self.device)
        residual = ops.embedding(ctx.token_ids, self.embedding)
        x = None
        for r, run in enumerate(self.plan.order):
            ctx.run = r
            layer = self.layers[run.layer]
            x = layer.block.forward(layer, x, residual, ctx)
        if logit_rows is not None and logit_rows.numel() == 0:  # the step only filled the cache
            return torch.empty((0, self.plan.head.vocab_size), dtype=torch.float32, device=self.device)
        h = self.final_norm.forward(norm_input(self.final_norm, x), residual, self.dtype, rows=logit_rows)
        return ops.linear(h, self.head, out_dtype=torch.float32)
