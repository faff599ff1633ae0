"""What every architecture's typed configuration has in common.

An architecture brings its own subclass with the keys of its config.json (the
Llama decoder's is config/llama.py) and registers it with its spec builder
(config/registry.py); nothing else in the package names an architecture's keys.
"""

from __future__ import annotations

from dataclasses import dataclass


class ConfigError(ValueError):
    """config.json is missing a key or asks for something the engine does not do."""


@dataclass(frozen=True)
class ModelConfig:
    """What every architecture's configuration has in common."""

    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    max_position_embeddings: int
    torch_dtype: str

    def to_hf_dict(self) -> dict:
        raise NotImplementedError
