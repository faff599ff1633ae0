"""One registry from the architecture's name in config.json to its model.

The reference keeps a set of supported names and imports the model class
directly (pagedllm/model/loader.py:14, :24-30); here an entry carries the typed
configuration class and the function that turns a configuration into a
`ModelSpec`.  Registering another architecture is one call of
`register_architecture`.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

from .model import ConfigError, ModelConfig


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: type
    build_spec: Callable[[ModelConfig], "ModelSpec"]  # noqa: F821


ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: type, build_spec: Callable) -> Architecture:
    if name in ARCHITECTURES:
        raise ValueError(f"architecture {name!r} is already registered")
    ARCHITECTURES[name] = Architecture(name, config_class, build_spec)
    return ARCHITECTURES[name]


def resolve_architecture(hf_config: dict) -> Architecture:
    """The first of config.json's `architectures` that is registered."""
    names = hf_config.get("architectures") or []
    for n in names:
        if n in ARCHITECTURES:
            return ARCHITECTURES[n]
    raise ConfigError(f"unsupported architecture {names}; registered: {sorted(ARCHITECTURES)}")


def parse_model_config(hf_config: dict) -> tuple[Architecture, ModelConfig]:
    arch = resolve_architecture(hf_config)
    return arch, arch.config_class.from_hf_dict(hf_config, architecture=arch.name)


def _register_builtin() -> None:
    from ..models.llama import llama_spec
    from .llama import LlamaConfig
    if "LlamaForCausalLM" not in ARCHITECTURES:
        register_architecture("LlamaForCausalLM", LlamaConfig, llama_spec)


_register_builtin()
