"""Things several parts of one model share: position tables, built once per (spec, device)."""

from __future__ import annotations

from tandem_b200.config.plan import PositionSpec
from tandem_b200.registry import part

_tables: dict = {}


def position_encoding(spec: PositionSpec, device):
    key = (spec, str(device))
    if key not in _tables:
        _tables[key] = part("position", spec.kind)(spec, device)
    return _tables[key]


def clear() -> None:
    _tables.clear()
