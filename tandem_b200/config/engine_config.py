"""Engine options, named as 12vivi/tandem names them (python/tandem/config.py:37-81).

Options of tandem that belong to parts this engine does not have (prefix cache, host KV tier,
attention backend choice, speculative decoding, hybrid MoE) are left out.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

_DTYPES = {"float32": "float32", "fp32": "float32", "bfloat16": "bfloat16", "bf16": "bfloat16", "auto": "auto"}


@dataclass
class EngineConfig:
    model: str  # folder with config.json and *.safetensors
    device: str = "cuda:0"
    dtype: str = "auto"  # "auto" | "bfloat16" | "float32"; auto = bfloat16 (python/tandem/utils.py:28-36)
    max_num_seqs: int = 64
    max_num_batched_tokens: int = 2048  # token budget of one step (chunked prefill)
    schedule_policy: str = "prefill_first"  # or "decode_first" (python/tandem/scheduler/scheduler.py:93-97)
    max_model_len: Optional[int] = None  # default min(max_position_embeddings, 32768) (llm_engine.py:55)
    block_size: int = 16  # tokens per KV page
    num_kv_blocks: Optional[int] = None  # pages per cache group; overrides kv_cache_memory_gb
    kv_cache_memory_gb: float = 1.0
    seed: int = 0
    cuda_graph: bool = True  # decode-only steps, and short steps with prompt portions, replay CUDA graphs
    cuda_graph_max_bs: int = 64
    cuda_graph_capture_at_start: bool = False  # capture every bucket when the engine is built (as the reference does) instead of at its first step
    small_batch_gemv: bool = True  # False: the library runs every bfloat16 product (cli.py:35-36 of the reference; process-wide)
    overlap_schedule: bool = True  # launch step N before step N-1's tokens reach the host (config.py:64 of the reference)

    def __post_init__(self) -> None:
        if self.dtype not in _DTYPES:
            raise ValueError(f"unknown dtype {self.dtype!r}; choose from {sorted(set(_DTYPES))}")
        self.dtype = _DTYPES[self.dtype]
        if self.schedule_policy not in ("prefill_first", "decode_first"):
            raise ValueError(f"unknown scheduling policy {self.schedule_policy!r}")
        for name in ("max_num_seqs", "max_num_batched_tokens", "block_size"):
            if getattr(self, name) <= 0:
                raise ValueError(f"{name} must be positive")

    @property
    def resolved_dtype(self) -> str:
        return "bfloat16" if self.dtype == "auto" else self.dtype
