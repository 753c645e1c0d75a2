"""tandem_b200: a single-GPU Qwen3-dense inference engine for NVIDIA B200 (sm_100a).

    from tandem_b200 import LLM, SamplingParams
    out = LLM(model="path/to/folder").generate([[1, 2, 3]], SamplingParams(max_tokens=8, temperature=0.0))

The public names follow 12vivi/tandem's (python/tandem/__init__.py:6-18).
"""

from tandem_b200.config.engine_config import EngineConfig
from tandem_b200.sampling.params import SamplingParams

__version__ = "0.1.0"
__all__ = ["EngineConfig", "SamplingParams", "LLMEngine", "LLM"]


def __getattr__(name):  # keeps `import tandem_b200` free of CUDA work
    if name in ("LLMEngine", "LLM"):
        from tandem_b200.engine import llm_engine

        return getattr(llm_engine, name)
    raise AttributeError(name)
