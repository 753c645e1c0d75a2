"""Put a model, its cache manager and its step function together.

``load_model`` goes from a model folder to a decoder through the architecture registry (the
model class is chosen by config.json, nowhere else); ``build_executor`` sizes the cache pool and
wires manager, storage and executor.  Generation, trace replay, the benchmark and the tests all
build the engine through these two functions.
"""

from __future__ import annotations

from typing import Any, Optional

import torch

from tandem_b200.cache.manager import CacheManager
from tandem_b200.cache.storage import CacheStorage
from tandem_b200.config.model_config import read_config_json
from tandem_b200.config.plan import ModelPlan
from tandem_b200.engine.executor import Executor
from tandem_b200.models.decoder import Decoder
from tandem_b200.registry import resolve_architecture
from tandem_b200.weights.loader import SafetensorsFolder, TensorDict, TensorSource

DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError(f"the engine runs on a CUDA device only (there is no CPU path), got {device}")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available: the engine cannot run")
    return device


def load_model(folder: str, dtype: str = "bfloat16", device="cuda:0") -> tuple[Decoder, Any]:
    """Model folder (config.json + *.safetensors) -> (decoder, typed configuration)."""
    cfg_dict = read_config_json(folder)
    arch = resolve_architecture(cfg_dict)
    cfg = arch.config_class.from_dict(cfg_dict)
    return Decoder(arch.build_plan(cfg), SafetensorsFolder(folder), DTYPES[dtype], require_cuda(device)), cfg


def random_model(config: dict, seed: int = 0, dtype: str = "bfloat16", device="cuda:0",
                 num_layers: Optional[int] = None, stored_dtype: Optional[str] = None) -> tuple[Decoder, Any]:
    """A model with seeded random weights made on the device, without a folder on disk (what
    ``write_random_model`` would store, drawn by the device's generator).  ``num_layers`` keeps
    only the first layers of the configuration.  ``stored_dtype``: the type the weights are drawn
    in before they are cast to ``dtype`` ("bfloat16" gives a float32 model the very numbers a
    bfloat16 model of the same seed has)."""
    arch = resolve_architecture(config)
    if num_layers is not None:
        config = dict(config, num_hidden_layers=num_layers)
    cfg = arch.config_class.from_dict(config)
    device = require_cuda(device)
    source = _Lazy(arch.random_weights(cfg, seed, str(device), DTYPES[stored_dtype or dtype]), "<random weights>")
    return Decoder(arch.build_plan(cfg), source, DTYPES[dtype], device), cfg


class _Lazy(TensorSource):
    """Tensors drawn one by one as the loader asks for them, in file order."""

    def __init__(self, iterator, where: str) -> None:
        self.where, self._it, self._held = where, iterator, {}

    def shapes(self):
        return None  # generated to fit the model: nothing to check

    def get(self, name: str) -> torch.Tensor:
        while name not in self._held:
            n, t = next(self._it)
            self._held[n] = t
        return self._held.pop(name)


def kv_bytes_per_token(decoder: Decoder) -> int:
    elem = torch.empty((), dtype=decoder.dtype).element_size()
    return sum(2 * n.num_kv_heads * n.head_dim * elem for n in decoder.kv_needs() if n is not None)


def build_executor(decoder: Decoder, page_size: int = 16, num_pages: Optional[int] = None,
                   cache_gb: float = 1.0, max_requests: int = 64) -> Executor:
    """Size the pool (``num_pages`` per cache group, or what ``cache_gb`` GiB hold:
    python/tandem/engine/llm_engine.py:78-80 of 12vivi/tandem) and build manager, storage, executor."""
    if num_pages is None:
        per_page = max(1, kv_bytes_per_token(decoder) * page_size)
        num_pages = int(cache_gb * 2**30 // per_page)
        if num_pages <= 0:
            raise ValueError(f"kv cache of {cache_gb} GiB holds no page of {per_page} bytes")
    kv_needs = decoder.kv_needs()
    manager = CacheManager(kv_needs, page_size, num_pages, max_requests)
    storage = CacheStorage(manager, kv_needs, decoder.cache_sources(), decoder.state_needs(), decoder.dtype,
                           decoder.device, users=decoder.cache_users)
    return Executor(decoder, manager, storage)
