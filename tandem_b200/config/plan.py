"""The model plan: what an architecture hands to the generic decoder.

A plan is data.  It lists the layers (each a block arrangement and the parts it arranges under
slot names of its own: norms, mixers, feed-forwards, every one a *spec*, a kind name plus the
sizes and constants that part takes), and the order in which the layers run.  The order is a list of :class:`RunStep`: it may name a
layer twice (the second run gets a cache of its own) or let a run read the cache that an
earlier run wrote (``cache_of``), in which case it writes none.

A spec never says which model it belongs to; parts are looked up by ``kind`` in
``tandem_b200.registry``.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional


@dataclass(frozen=True)
class WeightSource:
    """One checkpoint tensor copied into rows [row_start, row_start + rows) of a parameter."""

    name: str
    row_start: int = 0
    rows: Optional[int] = None  # None: the whole parameter


@dataclass(frozen=True)
class ParamSpec:
    """A parameter a part owns.

    role "matrix": a GEMM operand or embedding table, held in the model dtype.
    role "vector": a small tensor (norm weight), always held in float32.
    role "table_int": integers, held as int32.
    """

    shape: tuple
    sources: tuple  # of WeightSource
    role: str = "matrix"


@dataclass(frozen=True)
class PartSpec:
    """Base of every spec: ``kind`` picks the implementation in the registry, within the spec's
    ``family`` ("mixer", "feed_forward", "norm", "position")."""

    kind: str
    family = None  # set by the base class of each family


@dataclass(frozen=True)
class NormSpec(PartSpec):
    family = "norm"
    size: int = 0
    eps: float = 1e-6
    weight: str = ""  # checkpoint tensor name


@dataclass(frozen=True)
class PositionSpec(PartSpec):
    """kind "rope": rotate_half rotary encoding over the first ``rotary_dim`` dims of a head.
    kind "none": no position encoding."""

    family = "position"
    rotary_dim: int = 0
    theta: float = 10000.0
    max_position: int = 0


@dataclass(frozen=True)
class MixerSpec(PartSpec):
    family = "mixer"
    prefix: str = ""  # checkpoint name prefix, e.g. "model.layers.3.self_attn"


@dataclass(frozen=True)
class AttentionSpec(MixerSpec):
    hidden_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 1.0
    qk_norm: bool = False
    qk_norm_eps: float = 1e-6
    window: Optional[int] = None  # keys a query sees, itself included; None: all
    position: PositionSpec = PositionSpec("none")


@dataclass(frozen=True)
class FeedForwardSpec(PartSpec):
    family = "feed_forward"
    prefix: str = ""


@dataclass(frozen=True)
class GatedMLPSpec(FeedForwardSpec):
    hidden_size: int = 0
    intermediate_size: int = 0
    activation: str = "silu"


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the kind of its block arrangement and the parts that arrangement works with, as
    (slot name, family, spec).  Which slots there are is the arrangement's business: "prenorm" has
    ``mixer_norm``, ``mixer``, ``feed_forward_norm`` and ``feed_forward``; another arrangement may
    have four norms, no feed-forward, or two mixers side by side."""

    block: str
    parts: tuple

    @classmethod
    def of(cls, block: str, **slots: PartSpec) -> "LayerSpec":
        """``LayerSpec.of("prenorm", mixer=..., feed_forward=..., mixer_norm=..., feed_forward_norm=...)``:
        the family of each part is the one its spec class belongs to."""
        for name, spec in slots.items():
            if getattr(spec, "family", None) is None:
                raise TypeError(f"slot {name!r}: {type(spec).__name__} belongs to no part family "
                                "(derive it from MixerSpec, FeedForwardSpec, NormSpec or PositionSpec)")
        return cls(block, tuple((name, spec.family, spec) for name, spec in slots.items()))

    def slot(self, name: str) -> PartSpec:
        for slot, _, spec in self.parts:
            if slot == name:
                return spec
        raise KeyError(f"the layer has no slot {name!r} (it has {[s for s, _, _ in self.parts]})")

    def with_slot(self, name: str, spec: PartSpec) -> "LayerSpec":
        """A copy in which the slot holds ``spec`` (put behind the others if the slot is new)."""
        entry = (name, spec.family, spec)
        if any(slot == name for slot, _, _ in self.parts):
            return LayerSpec(self.block, tuple(entry if slot == name else (slot, fam, sp) for slot, fam, sp in self.parts))
        return LayerSpec(self.block, self.parts + (entry,))

    def of_family(self, family: str) -> list:
        """(slot name, spec) of the layer's parts of one family, in the order they were given."""
        return [(slot, spec) for slot, fam, spec in self.parts if fam == family]


@dataclass(frozen=True)
class RunStep:
    layer: int
    cache_of: Optional[int] = None  # index into ModelPlan.order of the run whose cache is read


@dataclass(frozen=True)
class EmbeddingSpec:
    """Start of the residual stream: ``scale * table[token]``, plus ``positions[position]`` where
    the model has a learned table of absolute positions (a checkpoint tensor [max_position, hidden])."""

    vocab_size: int
    hidden_size: int
    weight: str
    scale: float = 1.0
    positions: Optional[str] = None


@dataclass(frozen=True)
class HeadSpec:
    """Logits = ``scale * (h @ weight^T)``, then ``softcap * tanh(logits / softcap)`` where a cap is given."""

    vocab_size: int
    hidden_size: int
    weight: Optional[str]  # None: tied to the embedding table
    scale: float = 1.0
    softcap: Optional[float] = None


@dataclass(frozen=True)
class ModelPlan:
    embedding: EmbeddingSpec
    layers: tuple  # of LayerSpec
    order: tuple  # of RunStep
    final_norm: NormSpec
    head: HeadSpec
    max_position: int
    ignored_weights: tuple = ()  # regex patterns of checkpoint names that may be present and unused
    eos_token_ids: tuple = ()

    def __post_init__(self) -> None:
        for i, run in enumerate(self.order):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {run.layer}, the plan has {len(self.layers)}")
            if run.cache_of is not None:
                if not 0 <= run.cache_of < i:
                    raise ValueError(f"order[{i}].cache_of must name an earlier run, got {run.cache_of}")
                if self.order[run.cache_of].cache_of is not None:
                    raise ValueError(f"order[{i}].cache_of names a run that itself reads another run's cache")
