"""The generic decoder: embedding, the plan's runs in order, final norm, output head.

It is built from a :class:`~tandem_b200.config.plan.ModelPlan` and a source of checkpoint
tensors, looks every part up by kind in the registry, and knows no architecture by name.  The
loop is the one of 12vivi/tandem's python/tandem/models/llama_family.py:86-116 with the layer
order read from the plan instead of ``range(num_layers)``, and with the parts of a layer read
from the plan too: a layer is whatever its block arrangement declares as slots.
"""

from __future__ import annotations

from typing import Any, Optional

import torch

from tandem_b200.config.model_config import ConfigError
from tandem_b200.config.plan import ModelPlan, ParamSpec, WeightSource
from tandem_b200.kernels import deferred, ops
from tandem_b200.parts.base import StepContext
from tandem_b200.registry import part
from tandem_b200.weights.loader import TensorSource, load_parameters


class Layer:
    """A built layer: its arrangement and its parts, each also an attribute under its slot name."""

    def __init__(self, block: Any, parts: dict) -> None:
        self.block, self.parts = block, parts
        self.__dict__.update(parts)


def check_slots(index: int, layer_spec, block_class) -> None:
    """The layer's parts against what its arrangement declares (``slots``: name -> family, all
    needed; ``optional_slots``: likewise, may be absent)."""
    needed = dict(getattr(block_class, "slots", {}))
    allowed = dict(needed, **getattr(block_class, "optional_slots", {}))
    given = {slot: family for slot, family, _ in layer_spec.parts}
    missing = sorted(set(needed) - set(given))
    unknown = sorted(set(given) - set(allowed))
    wrong = sorted(s for s in given if s in allowed and allowed[s] != given[s])
    if missing or unknown or wrong:
        raise ConfigError(f"layer {index}: the {layer_spec.block!r} arrangement takes the slots {allowed}; "
                          f"missing {missing}, unknown {unknown}, of another family {wrong}")


class Decoder:
    def __init__(self, plan: ModelPlan, source: TensorSource, dtype: torch.dtype, device) -> None:
        self.plan, self.dtype, self.device = plan, dtype, torch.device(device)
        e, h = plan.embedding, plan.head
        params: dict[str, ParamSpec] = {"embedding": ParamSpec((e.vocab_size, e.hidden_size), (WeightSource(e.weight),))}
        if e.positions is not None:
            params["positions"] = ParamSpec((plan.max_position, e.hidden_size), (WeightSource(e.positions),))
        for i, layer in enumerate(plan.layers):
            check_slots(i, layer, part("block", layer.block))
            for slot, family, spec in layer.parts:
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
        self.positions = tensors.get("positions")
        self.head = tensors.get("head", self.embedding)  # tied: llama_family.py:108
        self.layers = []
        for i, layer in enumerate(plan.layers):
            built = {}
            for slot, family, spec in layer.parts:
                built[slot] = part(family, spec.kind)(spec, weights_of(f"layers.{i}.{slot}."), dtype, self.device)
                if family == "mixer":
                    built[slot].slot_name = slot  # how the mixer names itself when it asks for its cache
            self.layers.append(Layer(part("block", layer.block)(), built))
        self.final_norm = part("norm", plan.final_norm.kind)(plan.final_norm, weights_of("final_norm."), dtype,
                                                             self.device)
        self.num_parameters = sum(t.numel() for t in tensors.values())
        self.parameter_bytes = sum(t.numel() * t.element_size() for t in tensors.values())
        # Who keeps a cache: every mixer of every run, in running order.  The cache manager and the
        # storage number their entries by position in this list.
        self.cache_users = [(r, slot) for r, run in enumerate(plan.order)
                            for slot, _ in plan.layers[run.layer].of_family("mixer")]

    def mixers(self) -> list:
        """Every mixer of the model, once each, in layer order."""
        return [p for layer, spec in zip(self.layers, self.plan.layers) for slot, _ in spec.of_family("mixer")
                for p in (layer.parts[slot],)]

    def _mixer_spec(self, user: int):
        run, slot = self.cache_users[user]
        return self.plan.layers[self.plan.order[run].layer].slot(slot)

    # what the cache manager has to provide for each cache user
    def kv_needs(self) -> list:
        out = []
        for user, (run, _) in enumerate(self.cache_users):
            spec = self._mixer_spec(user)
            shared = self.plan.order[run].cache_of is not None
            out.append(None if shared else part("mixer", spec.kind).kv_need(spec))
        return out

    def state_needs(self) -> list:
        return [part("mixer", self._mixer_spec(u).kind).state_need(self._mixer_spec(u)) for u in range(len(self.cache_users))]

    def cache_sources(self) -> list:
        """Per cache user: the user whose keys and values it reads instead of its own (a run with
        ``cache_of`` reads, slot by slot, what the named earlier run wrote), else None."""
        index = {key: u for u, key in enumerate(self.cache_users)}
        return [index.get((self.plan.order[run].cache_of, slot)) if self.plan.order[run].cache_of is not None else None
                for run, slot in self.cache_users]

    def forward(self, ctx: StepContext, logit_rows: Optional[torch.Tensor]) -> torch.Tensor:
        """Logits float32 [R, vocab] at the rows ``logit_rows`` (int32 indices into the step's
        tokens; None: every token).  Runs only the tokens of the step, from the cache."""
        e, h = self.plan.embedding, self.plan.head
        if ctx.num_tokens == 0:
            return torch.empty((0, h.vocab_size), dtype=torch.float32, device=self.device)
        residual = ops.embedding(ctx.token_ids, self.embedding, scale=e.scale, positions=ctx.positions,
                                 position_table=self.positions)
        x = None
        for r, run in enumerate(self.plan.order):
            ctx.run = r
            layer = self.layers[run.layer]
            if not getattr(layer.block, "takes_deferred", False):
                x = deferred.tensor(x)  # the arrangement before may have left its last product pending
            x = layer.block.forward(layer, x, residual, ctx)
        if logit_rows is not None and logit_rows.numel() == 0:  # the step only filled the cache
            return torch.empty((0, h.vocab_size), dtype=torch.float32, device=self.device)
        if not getattr(self.final_norm, "takes_deferred", False):
            x = deferred.tensor(x)
        hidden = self.final_norm.forward(x, residual, self.dtype, rows=logit_rows)
        logits = ops.linear(hidden, self.head, out_dtype=torch.float32)
        if h.scale != 1.0 or h.softcap is not None:
            ops.scale_softcap(logits, h.scale, h.softcap)
        return logits
