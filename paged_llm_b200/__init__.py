"""A paged LLM inference engine for one NVIDIA B200 and the Llama dense decoder."""

from .config import EngineConfig, SamplingParams

__all__ = ["EngineConfig", "SamplingParams", "LLMEngine"]
__version__ = "0.1.0"


def __getattr__(name):
    if name == "LLMEngine":
        from .engine.llm_engine import LLMEngine
        return LLMEngine
    raise AttributeError(name)
