"""Shared fixtures: tiny random-weight Qwen3 folders (made in temporary folders) and helpers.

Tests marked ``gpu`` need a CUDA device; everything else runs on the CPU."""

from __future__ import annotations

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)

# Two tiny configurations that differ in every size and option, and a third with a window.
TINY_A = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=2, head_dim=16, intermediate_size=192, vocab_size=512,
              rope_theta=10000.0, rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=256)
TINY_B = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=3, hidden_size=96,
              num_attention_heads=6, num_key_value_heads=2, head_dim=32, intermediate_size=256, vocab_size=1000,
              rope_theta=1000000.0, rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=512)
TINY_C = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=4, hidden_size=120,
              num_attention_heads=6, num_key_value_heads=3, head_dim=48, intermediate_size=200, vocab_size=777,
              rope_theta=500000.0, rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=384,
              use_sliding_window=True, sliding_window=20, max_window_layers=2)
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C}
PAGE = {"A": 4, "B": 8, "C": 16}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def tiny_folder(tmp_path_factory):
    """name ("A" | "B" | "C") -> model folder with bfloat16-representable random weights."""
    from tandem_b200.weights.random_init import write_random_model

    made = {}

    def make(name: str, std: float = 0.05) -> str:
        key = (name, std)
        if key not in made:
            folder = str(tmp_path_factory.mktemp(f"tiny{name}"))
            write_random_model(TINY[name], folder, seed=11 + ord(name), dtype="bfloat16", std=std)
            made[key] = folder
        return made[key]

    return make


def random_tokens(seed: int, n: int, vocab: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
