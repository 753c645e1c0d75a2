"""What every part is given, and the interfaces parts implement.

A *part* is built from its spec (sizes and constants), its weights (already on the device, by the
local names its ``params`` declared) and the model dtype.  It never learns which model it is in.
During a step it is handed a :class:`StepContext`: the flattened batch and, through it, the
cache of the run in flight.

Interfaces (duck-typed; these base classes only document them and give the defaults):

``Mixer``         ``params(spec)``, ``kv_need(spec)``, ``state_need(spec)``, ``forward(x, ctx) -> y``,
                  optionally ``step_arrays(ctx, out)``
``FeedForward``   ``params(spec)``, ``forward(x, ctx) -> y``
``Norm``          ``params(spec)``, ``forward(x, residual, out_dtype, rows=None) -> y`` (adds x into
                  the float32 residual in place, then normalises it)
``PositionEncoding``  built from its spec alone; what it offers is up to the mixers that use it
``Block``         ``forward(layer, x, residual, ctx) -> x`` (the arrangement of norms, mixer and
                  feed-forward around the residual stream)
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from tandem_b200.cache.manager import KVNeed
from tandem_b200.config.plan import ParamSpec


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size that a mixer keeps: one row of ``shape`` per live request."""

    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class KVView:
    """The paged cache of one run, as a mixer sees it during a step."""

    k: torch.Tensor  # [pages, kv heads, page_size, head_dim]
    v: torch.Tensor
    block_table: torch.Tensor  # int32 [B, max_pages] of the run's group; -1 where a page was given back
    slots: torch.Tensor  # int32 [T]: page * page_size + offset of each token of the step
    page_size: int
    writable: bool  # False: the run reads the cache another run wrote


@dataclass
class StepContext:
    """One step's batch: B requests, T tokens in all, request after request."""

    dtype: torch.dtype
    device: torch.device
    num_tokens: int
    num_seqs: int
    token_ids: torch.Tensor  # int32 [T]
    positions: torch.Tensor  # int32 [T], position of each token in its request
    seq_of_token: torch.Tensor  # int32 [T], index of the token's request in this step
    cu_seqlens: torch.Tensor  # int32 [B + 1], offsets of the requests' tokens
    seq_starts: torch.Tensor  # int32 [B], tokens each request had stored before this step
    state_slots: torch.Tensor  # int32 [B], row of each request in the state tensors
    host_starts: list  # the same numbers on the host
    host_lens: list  # new tokens per request
    host_slots: list
    max_new: int  # longest portion in the step
    max_total: int  # longest request after the step (start + new)
    storage: Any = None  # CacheStorage
    page_size: int = 0
    extras: dict = field(default_factory=dict)  # key -> int32 device array a mixer asked for (Mixer.step_arrays)
    tables: dict = field(default_factory=dict)  # group -> (block_table, slots)
    run: int = 0  # position in ModelPlan.order of the run in flight
    # The step is captured into, or replayed from, a CUDA graph that also takes prompt portions: num_tokens and
    # num_seqs are the graph's capacities (rows beyond the real tokens are padding), and the arrays of
    # ``Mixer.step_arrays`` must keep the layout of their capacity whatever the step brings.
    static_layout: bool = False
    scratch: dict = field(default_factory=dict)  # per-step values parts may share (keyed by them)

    def kv(self, mixer: Any = None) -> KVView:
        """The paged cache of the mixer that asks (``ctx.kv(self)``), in the run in flight.  A layer
        with a single mixer may leave the argument out."""
        return self.storage.view(self.storage.user(self.run, mixer), self)

    def state(self, mixer: Any = None) -> torch.Tensor:
        """[max requests + 1, *shape] tensor of the asking mixer's per-request state in the run in
        flight; the last row belongs to no request (rows that pad a captured batch point there)."""
        return self.storage.state[self.storage.user(self.run, mixer)]


class PlanTooLarge(RuntimeError):
    """Raised from ``Mixer.step_arrays`` under ``ctx.static_layout``: this step's arrays do not fit the room
    that the mixer asked for, so the step runs without a CUDA graph."""


class Mixer:
    @staticmethod
    def params(spec) -> dict[str, ParamSpec]:
        return {}

    @staticmethod
    def kv_need(spec) -> Optional[KVNeed]:
        return None

    @staticmethod
    def state_need(spec) -> Optional[StateNeed]:
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError

    # Optional: ``step_arrays(self, ctx, out)`` is called once per step, before anything runs, with
    # the host side of the batch (ctx.host_starts, ctx.host_lens, ...).  It may add integer arrays
    # to ``out`` under keys of its own (skipping keys that are already there); they travel to the
    # device with the batch description and appear as ``ctx.extras[key]`` in ``forward``.
    # A mixer that does so tells CUDA graphs how large the arrays can get:
    # ``step_array_capacity(self, bucket, max_model_len, page_size, out)`` for steps of up to ``bucket`` single
    # tokens, and (optional) ``mixed_step_array_capacity(self, tokens, seqs, max_model_len, page_size, out)``
    # for steps of up to ``tokens`` tokens of up to ``seqs`` requests (``ctx.static_layout``); out[key] = entries.
    # ``capturable = True``: ``forward`` of a step of single tokens only launches kernels and reads the batch from
    # the context's device arrays, never from its host-side lists; ``capturable_portions = True``: the same holds
    # for steps in which requests bring several tokens.


class FeedForward:
    @staticmethod
    def params(spec) -> dict[str, ParamSpec]:
        return {}

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Norm:
    @staticmethod
    def params(spec) -> dict[str, ParamSpec]:
        return {}

    def forward(self, x: Optional[torch.Tensor], residual: torch.Tensor, out_dtype: torch.dtype,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError
