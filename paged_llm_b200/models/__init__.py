from .causal_lm import CacheSlot, CausalLM, build_model
from .llama import llama_spec

__all__ = ["CacheSlot", "CausalLM", "build_model", "llama_spec"]
