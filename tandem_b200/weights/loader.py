"""Fill a model's parameters from checkpoint tensors, by name.

The model says what it needs as ``{parameter name: ParamSpec}``; each ParamSpec lists the
checkpoint tensors that make it up (one, or several stacked by rows: q/k/v -> qkv, gate/up ->
gate_up, as python/tandem/models/loader.py:22-57 fuses them).  Everything is checked against the
checkpoint's header before a byte is copied, and all faults are reported together in one
:class:`WeightError`: missing tensors, unexpected tensors, wrong shapes.

Held dtypes: "matrix" parameters in the model dtype (bfloat16 when serving, float32 on the
32-bit path); "vector" parameters (norm weights) always in float32, so a tensor the checkpoint
stores in 32 bits keeps them; "table_int" parameters as int32.
"""

from __future__ import annotations

import glob
import os
import re
from typing import Iterable, Iterator, Optional

import torch

from tandem_b200.config.plan import ParamSpec


class WeightError(RuntimeError):
    """The checkpoint does not fit the model.  ``missing``, ``unexpected`` and ``wrong_shape``
    (name, found, wanted) carry the details that the message lists."""

    def __init__(self, where: str, missing: list, unexpected: list, wrong_shape: list) -> None:
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        lines = [f"checkpoint {where} does not fit the model:"]
        if missing:
            lines.append(f"  {len(missing)} missing: " + ", ".join(missing[:8]) + (" ..." if len(missing) > 8 else ""))
        if unexpected:
            lines.append(f"  {len(unexpected)} unexpected: " + ", ".join(unexpected[:8])
                         + (" ..." if len(unexpected) > 8 else ""))
        for name, found, wanted in wrong_shape[:8]:
            lines.append(f"  wrong shape: {name} is {tuple(found)}, the model wants {tuple(wanted)}")
        if len(wrong_shape) > 8:
            lines.append(f"  ... and {len(wrong_shape) - 8} more wrong shapes")
        super().__init__("\n".join(lines))


# --------------------------------------------------------------------------- sources
class TensorSource:
    """Where checkpoint tensors come from."""

    where = "<memory>"

    def shapes(self) -> Optional[dict[str, tuple]]:
        """Name -> shape of every tensor held; None if the tensors are generated to fit."""
        raise NotImplementedError

    def get(self, name: str) -> torch.Tensor:
        raise NotImplementedError

    def close(self) -> None:
        pass


class SafetensorsFolder(TensorSource):
    """Every ``*.safetensors`` file of a folder, sorted (python/tandem/models/loader.py:67-78)."""

    def __init__(self, folder: str) -> None:
        from safetensors import safe_open

        self.where = folder
        files = sorted(glob.glob(os.path.join(folder, "*.safetensors")))
        if not files:
            raise FileNotFoundError(f"no *.safetensors files in {folder}")
        self._handles = [safe_open(p, framework="pt", device="cpu") for p in files]
        self._owner: dict[str, int] = {}
        self._shapes: dict[str, tuple] = {}
        for i, h in enumerate(self._handles):
            for name in h.keys():
                self._owner[name] = i
                self._shapes[name] = tuple(h.get_slice(name).get_shape())

    def shapes(self) -> dict[str, tuple]:
        return self._shapes

    def get(self, name: str) -> torch.Tensor:
        return self._handles[self._owner[name]].get_tensor(name)

    def close(self) -> None:
        self._handles = []


class TensorDict(TensorSource):
    """Tensors already in memory (the random-weights mode without a folder)."""

    def __init__(self, tensors: Iterable[tuple[str, torch.Tensor]], where: str = "<memory>") -> None:
        self.where = where
        self._tensors = dict(tensors)

    def shapes(self) -> dict[str, tuple]:
        return {n: tuple(t.shape) for n, t in self._tensors.items()}

    def get(self, name: str) -> torch.Tensor:
        return self._tensors.pop(name)  # handed over: the caller's copy is the only one kept


# --------------------------------------------------------------------------- loading
_HELD = {"vector": torch.float32, "table_int": torch.int32}


def check(params: dict[str, ParamSpec], have: dict[str, tuple], ignored: tuple, where: str) -> None:
    missing, wrong, used = [], [], set()
    for pname, spec in params.items():
        for src in spec.sources:
            used.add(src.name)
            if src.name not in have:
                missing.append(src.name)
                continue
            rows = spec.shape[0] if src.rows is None else src.rows
            wanted = (rows,) + tuple(spec.shape[1:])
            if tuple(have[src.name]) != wanted:
                wrong.append((src.name, have[src.name], wanted))
    patterns = [re.compile(p) for p in ignored]
    unexpected = sorted(n for n in have if n not in used and not any(p.search(n) for p in patterns))
    if missing or wrong or unexpected:
        raise WeightError(where, sorted(set(missing)), unexpected, wrong)


def load_parameters(params: dict[str, ParamSpec], source: TensorSource, dtype: torch.dtype, device: str,
                    ignored: tuple = ()) -> dict[str, torch.Tensor]:
    """-> {parameter name: tensor on ``device``}.  Raises WeightError before copying anything."""
    have = source.shapes()
    if have is not None:
        check(params, have, ignored, source.where)
    out: dict[str, torch.Tensor] = {}
    for pname, spec in params.items():
        held = _HELD.get(spec.role, dtype)
        if len(spec.sources) == 1 and spec.sources[0].rows is None:
            out[pname] = source.get(spec.sources[0].name).to(device=device, dtype=held).contiguous()
            continue
        t = torch.empty(spec.shape, dtype=held, device=device)
        for src in spec.sources:
            rows = spec.shape[0] if src.rows is None else src.rows
            t[src.row_start: src.row_start + rows].copy_(source.get(src.name).to(device=device, dtype=held))
        out[pname] = t
    source.close()
    return out
