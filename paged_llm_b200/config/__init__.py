from .engine import EngineConfig
from .model import ConfigError, LlamaConfig, ModelConfig, RopeScaling
from .registry import ARCHITECTURES, Architecture, parse_model_config, register_architecture, resolve_architecture
from .sampling import SamplingParams

__all__ = ["EngineConfig", "ConfigError", "LlamaConfig", "ModelConfig", "RopeScaling", "ARCHITECTURES",
           "Architecture", "parse_model_config", "register_architecture", "resolve_architecture", "SamplingParams"]
