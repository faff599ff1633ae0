from .engine import EngineConfig
from .llama import LlamaConfig, RopeScaling
from .model import ConfigError, ModelConfig
from .registry import ARCHITECTURES, Architecture, parse_model_config, register_architecture, resolve_architecture
from .sampling import SamplingParams

__all__ = ["EngineConfig", "ConfigError", "LlamaConfig", "ModelConfig", "RopeScaling", "ARCHITECTURES",
           "Architecture", "parse_model_config", "register_architecture", "resolve_architecture", "SamplingParams"]
