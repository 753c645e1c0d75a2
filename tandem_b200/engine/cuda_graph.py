"""CUDA graphs for decode-only steps (placeholder until the graph runner is wired)."""

from __future__ import annotations


class DecodeGraphs:
    @classmethod
    def maybe(cls, executor, max_batch: int, max_model_len: int):
        return None
