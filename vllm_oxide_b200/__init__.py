"""vllm_oxide_b200: a small, whole, single-GPU inference engine for Qwen3 (dense) on B200 (sm_100a).

    from vllm_oxide_b200 import LLM, EngineOptions, SamplingParams
"""
from .config.engine_options import EngineOptions
from .sampling.params import SamplingParams

__all__ = ["LLM", "EngineOptions", "SamplingParams", "RequestOutput"]


def __getattr__(name):
    if name in ("LLM", "RequestOutput"):
        from .engine import llm
        return getattr(llm, name)
    raise AttributeError(name)
