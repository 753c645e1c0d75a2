"""Typed view of a Qwen3 ``config.json``.

Every size and constant of the model comes from here; nothing below this file hard-codes one.
Keys and defaults follow python/tandem/model_config.py:90-145 of 12vivi/tandem; options that
the engine does not implement are rejected here instead of being computed wrongly.
"""

from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Optional


class ConfigError(ValueError):
    """config.json is missing a key, or asks for something the engine does not have."""


def _require(d: dict, key: str) -> Any:
    if key not in d or d[key] is None:
        raise ConfigError(f"config.json: required key {key!r} is missing")
    return d[key]


def _positive_int(d: dict, key: str, value: Any) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json: {key!r} must be a positive integer, got {value!r}")
    return value


@dataclass(frozen=True)
class Qwen3Config:
    """Qwen3 dense decoder (python/tandem/model_config.py:46-72, the keys that family reads)."""

    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    sliding_window: Optional[int] = None  # keys each windowed layer sees, None: every layer sees all
    max_window_layers: int = 0  # layers with index >= this are windowed (when sliding_window is set)
    layer_types: Optional[tuple] = None  # per layer "full_attention" | "sliding_attention"; overrides max_window_layers
    eos_token_ids: tuple = ()
    torch_dtype: Optional[str] = None
    extra: dict = field(default_factory=dict, compare=False)  # unread keys, kept for to_dict()

    # ---------------------------------------------------------------- derived
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def layer_window(self, layer: int) -> Optional[int]:
        if self.layer_types is not None:
            return self.sliding_window if self.layer_types[layer] == "sliding_attention" else None
        if self.sliding_window is None or layer < self.max_window_layers:
            return None
        return self.sliding_window

    # ---------------------------------------------------------------- reading
    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "Qwen3Config":
        arch = (d.get("architectures") or [None])[0] or d.get("model_type")
        hidden = _positive_int(d, "hidden_size", _require(d, "hidden_size"))
        nh = _positive_int(d, "num_attention_heads", _require(d, "num_attention_heads"))
        nkv = d.get("num_key_value_heads") or nh  # model_config.py:125
        head_dim = d.get("head_dim") or hidden // nh  # model_config.py:100-101
        _positive_int(d, "num_key_value_heads", nkv)
        _positive_int(d, "head_dim", head_dim)
        if nh % nkv:
            raise ConfigError(f"num_attention_heads ({nh}) must be a multiple of num_key_value_heads ({nkv})")
        if head_dim % 2:
            raise ConfigError(f"head_dim ({head_dim}) must be even for rotary position encoding")

        # transformers >= 5 writes rope settings under `rope_parameters` (model_config.py:103-113)
        rope_params = d.get("rope_parameters") if isinstance(d.get("rope_parameters"), dict) else None
        if rope_params:
            theta = float(rope_params.get("rope_theta") or d.get("rope_theta") or 10000.0)
            scaling = dict(rope_params)
        else:
            theta = float(d.get("rope_theta") or 10000.0)
            scaling = dict(d["rope_scaling"]) if d.get("rope_scaling") else None
        if scaling is not None:
            kind = scaling.get("rope_type", scaling.get("type", "default"))
            if kind != "default":
                raise ConfigError(f"rope scaling {kind!r} is not supported (only the default rotary encoding)")
        if d.get("attention_bias"):
            raise ConfigError("attention_bias=true is not supported (Qwen3 projections have no bias)")
        if d.get("quantization_config"):
            raise ConfigError("quantized checkpoints are not supported")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported (SwiGLU uses silu)")

        window = None
        if d.get("use_sliding_window"):
            window = _positive_int(d, "sliding_window", _require(d, "sliding_window"))
        first_window_layer = d.get("max_window_layers")
        layers = _positive_int(d, "num_hidden_layers", _require(d, "num_hidden_layers"))
        if first_window_layer is None:
            first_window_layer = layers if window is None else 0
        # newer config.json files name each layer's kind; where they do, that list decides
        layer_types = d.get("layer_types")
        if layer_types is not None:
            layer_types = tuple(layer_types)
            if len(layer_types) != layers:
                raise ConfigError(f"layer_types has {len(layer_types)} entries for {layers} layers")
            for kind in layer_types:
                if kind not in ("full_attention", "sliding_attention"):
                    raise ConfigError(f"layer type {kind!r} is not supported (full_attention or sliding_attention)")
            if "sliding_attention" in layer_types:
                window = _positive_int(d, "sliding_window", _require(d, "sliding_window"))
            else:
                window = None

        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))

        known = {
            "architectures", "model_type", "vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
            "num_key_value_heads", "head_dim", "intermediate_size", "rms_norm_eps", "rope_theta", "rope_scaling",
            "rope_parameters", "max_position_embeddings", "tie_word_embeddings", "attention_bias", "hidden_act",
            "use_sliding_window", "sliding_window", "max_window_layers", "eos_token_id", "torch_dtype", "dtype",
            "quantization_config", "layer_types",
        }
        return cls(
            architecture=arch,
            vocab_size=_positive_int(d, "vocab_size", _require(d, "vocab_size")),
            hidden_size=hidden,
            num_hidden_layers=layers,
            num_attention_heads=nh,
            num_key_value_heads=nkv,
            head_dim=head_dim,
            intermediate_size=_positive_int(d, "intermediate_size", _require(d, "intermediate_size")),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-6)),  # model_config.py:128
            rope_theta=theta,
            max_position_embeddings=_positive_int(d, "max_position_embeddings", d.get("max_position_embeddings", 4096)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            sliding_window=window,
            max_window_layers=int(first_window_layer),
            layer_types=layer_types,
            eos_token_ids=eos_ids,
            torch_dtype=d.get("torch_dtype") or d.get("dtype"),
            extra={k: v for k, v in d.items() if k not in known},
        )

    def to_dict(self) -> dict[str, Any]:
        """The config.json this configuration is read back from."""
        d: dict[str, Any] = dict(self.extra)
        d.update(
            architectures=[self.architecture],
            model_type="qwen3",
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            num_hidden_layers=self.num_hidden_layers,
            num_attention_heads=self.num_attention_heads,
            num_key_value_heads=self.num_key_value_heads,
            head_dim=self.head_dim,
            intermediate_size=self.intermediate_size,
            hidden_act="silu",
            rms_norm_eps=self.rms_norm_eps,
            rope_theta=self.rope_theta,
            max_position_embeddings=self.max_position_embeddings,
            tie_word_embeddings=self.tie_word_embeddings,
            attention_bias=False,
            use_sliding_window=self.sliding_window is not None,
            sliding_window=self.sliding_window,
            max_window_layers=self.max_window_layers,
        )
        if self.layer_types is not None:
            d["layer_types"] = list(self.layer_types)
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids) if len(self.eos_token_ids) > 1 else self.eos_token_ids[0]
        if self.torch_dtype:
            d["torch_dtype"] = self.torch_dtype
        return d


def read_config_json(folder: str) -> dict[str, Any]:
    path = os.path.join(folder, "config.json")
    if not os.path.isfile(path):
        raise FileNotFoundError(f"no config.json in {folder}")
    with open(path, encoding="utf-8") as f:
        d = json.load(f)
    gen = os.path.join(folder, "generation_config.json")  # model_config.py:151-157
    if os.path.isfile(gen):
        with open(gen, encoding="utf-8") as f:
            eos = json.load(f).get("eos_token_id")
        if eos is not None:
            have = d.get("eos_token_id")
            have = [] if have is None else ([have] if isinstance(have, int) else list(have))
            extra = [eos] if isinstance(eos, int) else list(eos)
            d["eos_token_id"] = sorted(set(have) | set(extra))
    return d
