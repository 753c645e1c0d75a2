"""Name -> implementation tables: architectures and the kinds of parts.

One registry for whole architectures (``config.json``'s ``architectures[0]`` or ``model_type``
-> configuration class + plan builder), and one per kind of part (mixer, feed-forward, norm,
position encoding, block arrangement).  Adding an architecture or a part is one ``register_*``
call; the decoder, cache manager, step function and scheduler never name a model.
12vivi/tandem keeps the same tables in python/tandem/model_config.py:11-24 and
python/tandem/models/__init__.py:8-14.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from tandem_b200.config.model_config import ConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any  # has from_dict(dict) and to_dict()
    build_plan: Callable[[Any], Any]  # config -> ModelPlan
    random_weights: Callable[..., Any]  # (config, seed, device, dtype) -> iterator of (name, tensor)


_ARCHITECTURES: dict[str, Architecture] = {}
_MODEL_TYPES: dict[str, str] = {}
_PARTS: dict[str, dict[str, Any]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}}


def register_architecture(arch: Architecture, model_types: tuple = ()) -> None:
    _ARCHITECTURES[arch.name] = arch
    for t in model_types:
        _MODEL_TYPES[t] = arch.name


def resolve_architecture(config: dict) -> Architecture:
    """The architecture a config.json names; NotImplementedError lists the known ones otherwise
    (python/tandem/model_config.py:91-95)."""
    _load_builtin()
    name = (config.get("architectures") or [None])[0]
    if name not in _ARCHITECTURES:
        name = _MODEL_TYPES.get(config.get("model_type", ""), name)
    if name not in _ARCHITECTURES:
        raise NotImplementedError(
            f"architecture {name!r} is not supported (supported: {sorted(_ARCHITECTURES)})"
        )
    return _ARCHITECTURES[name]


def supported_architectures() -> list[str]:
    _load_builtin()
    return sorted(_ARCHITECTURES)


def register_part(family: str, kind: str, implementation: Any) -> None:
    """family: "mixer" | "feed_forward" | "norm" | "position" | "block"."""
    if family not in _PARTS:
        raise KeyError(f"unknown part family {family!r} (have {sorted(_PARTS)})")
    _PARTS[family][kind] = implementation


def part(family: str, kind: str) -> Any:
    _load_builtin()
    try:
        return _PARTS[family][kind]
    except KeyError:
        raise ConfigError(f"no {family} of kind {kind!r} is registered (have {sorted(_PARTS[family])})") from None


_loaded = False


def _load_builtin() -> None:
    """Import the modules that register the built-in architecture and parts."""
    global _loaded
    if _loaded:
        return
    _loaded = True
    import tandem_b200.models.qwen3  # noqa: F401
    import tandem_b200.parts  # noqa: F401
