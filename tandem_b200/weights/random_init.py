"""Random-weights mode: a configuration and a seed -> a model folder.

The folder holds what a downloaded checkpoint holds (``config.json`` and ``model.safetensors``
with the architecture's own tensor names), so it is read back through the normal loader.
12vivi/tandem has no such mode in the library; its tests overwrite the parameters of a freshly
built model (tests/conftest.py:71-79).
"""

from __future__ import annotations

import json
import os
from typing import Any, Union

import torch

from tandem_b200.registry import resolve_architecture

_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def write_random_model(config: Union[dict, Any], folder: str, seed: int = 0, dtype: str = "bfloat16",
                       std: float = 0.02, norm_spread: float = 0.1) -> str:
    """Write ``folder/config.json`` and ``folder/model.safetensors``; returns the folder.

    ``config`` is a config.json dictionary or an architecture's configuration object.
    ``dtype`` is the storage type of every tensor; values stored as bfloat16 are exactly
    representable, so the 32-bit path and the bfloat16 path read the same numbers."""
    from safetensors.torch import save_file

    cfg_dict = config if isinstance(config, dict) else config.to_dict()
    arch = resolve_architecture(cfg_dict)
    cfg = arch.config_class.from_dict(cfg_dict)
    os.makedirs(folder, exist_ok=True)
    out = cfg.to_dict()
    out["torch_dtype"] = dtype
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(out, f, indent=1)
    tensors = {name: t.contiguous() for name, t in
               arch.random_weights(cfg, seed, "cpu", _STORE[dtype], std=std, norm_spread=norm_spread)}
    save_file(tensors, os.path.join(folder, "model.safetensors"), metadata={"format": "pt"})
    return folder
