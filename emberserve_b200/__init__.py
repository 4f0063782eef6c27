"""emberserve_b200: a small, whole inference engine for Qwen2.5 dense on one B200.

    from emberserve_b200 import LLM, SamplingParams
    out = LLM(model_dir, dtype="bfloat16").generate([[1, 2, 3]], SamplingParams.greedy(16))
"""

from emberserve_b200.config.engine import EngineConfig
from emberserve_b200.sampling.params import SamplingParams

__all__ = ["EngineConfig", "LLM", "LLMEngine", "SamplingParams"]


def __getattr__(name):  # the engine classes import torch-heavy modules: load them on demand
    if name == "LLM":
        from emberserve_b200.llm import LLM

        return LLM
    if name == "LLMEngine":
        from emberserve_b200.engine.llm_engine import LLMEngine

        return LLMEngine
    raise AttributeError(name)
