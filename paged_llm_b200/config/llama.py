"""Typed configuration of the Llama dense decoder, read from a checkpoint's config.json.

`LlamaConfig.from_hf_dict` reads the keys that the reference's
`LlamaConfig.from_hf` reads (pagedllm/model/llama.py:37-60) with the same
defaults.  Keys that the reference silently ignores although they change the
mathematics (`hidden_act`, `attention_bias`, `mlp_bias`) are checked here and an
unsupported value is an error, not a wrong result.
"""

from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field
from typing import Any

from .model import ConfigError, ModelConfig


@dataclass(frozen=True)
class RopeScaling:
    """Frequency rescaling of the rotary table (llama.py:86-97).  Only the
    'llama3' rule exists in the reference; 'default' means none."""

    rope_type: str
    factor: float
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192

    @classmethod
    def from_dict(cls, d: dict) -> "RopeScaling | None":
        kind = d.get("rope_type", d.get("type", "default"))
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise ConfigError(f"rope_type={kind!r} is not supported (default and llama3 only)")
        if "factor" not in d:
            raise ConfigError("rope scaling of type llama3 needs a 'factor'")
        return cls(
            rope_type=kind,
            factor=float(d["factor"]),
            low_freq_factor=float(d.get("low_freq_factor", 1.0)),
            high_freq_factor=float(d.get("high_freq_factor", 4.0)),
            original_max_position_embeddings=int(d.get("original_max_position_embeddings", 8192)),
        )

    def to_dict(self) -> dict:
        return asdict(self)



_REQUIRED = ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads")


@dataclass(frozen=True)
class LlamaConfig(ModelConfig):
    intermediate_size: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rms_norm_eps: float = 1e-5
    rope_theta: float = 10000.0
    rope_scaling: RopeScaling | None = None
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    extra: dict = field(default_factory=dict, compare=False, hash=False)

    # ---- reading ------------------------------------------------------------
    @classmethod
    def from_hf_dict(cls, cfg: dict[str, Any], architecture: str = "LlamaForCausalLM") -> "LlamaConfig":
        missing = [k for k in _REQUIRED if k not in cfg]
        if missing:
            raise ConfigError(f"config.json lacks required keys: {missing}")
        heads = int(cfg["num_attention_heads"])
        # Newer checkpoints nest theta and scaling under "rope_parameters"; older
        # ones have a top-level "rope_theta" and an optional "rope_scaling".
        rope = dict(cfg.get("rope_parameters") or cfg.get("rope_scaling") or {})
        theta = rope.pop("rope_theta", None) or cfg.get("rope_theta", 10000.0)
        head_dim = cfg.get("head_dim") or int(cfg["hidden_size"]) // heads
        self = cls(
            architecture=architecture,
            vocab_size=int(cfg["vocab_size"]),
            hidden_size=int(cfg["hidden_size"]),
            num_hidden_layers=int(cfg["num_hidden_layers"]),
            max_position_embeddings=int(cfg.get("max_position_embeddings", 4096)),
            torch_dtype=str(cfg.get("torch_dtype") or cfg.get("dtype") or "float16"),
            intermediate_size=int(cfg["intermediate_size"]),
            num_attention_heads=heads,
            num_key_value_heads=int(cfg.get("num_key_value_heads") or heads),
            head_dim=int(head_dim),
            rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-5)),
            rope_theta=float(theta),
            rope_scaling=RopeScaling.from_dict(rope),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            hidden_act=str(cfg.get("hidden_act", "silu")),
            extra={k: cfg[k] for k in ("attention_bias", "mlp_bias") if k in cfg},
        )
        self.validate()
        return self

    def validate(self) -> None:
        for name in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                     "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings"):
            if getattr(self, name) < 1:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads={self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even for rotary pairs")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act={self.hidden_act!r}: only 'silu' is implemented")
        for key in ("attention_bias", "mlp_bias"):
            if self.extra.get(key):
                raise ConfigError(f"{key}=true: projections with bias are not implemented")
        if not (self.rms_norm_eps > 0 and math.isfinite(self.rms_norm_eps)):
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")
        if not self.rope_theta > 0:
            raise ConfigError(f"rope_theta must be positive, got {self.rope_theta}")

    # ---- writing ------------------------------------------------------------
    def to_hf_dict(self) -> dict:
        d = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": self.hidden_act,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": self.torch_dtype,
        }
        return d

    @property
    def num_parameters(self) -> int:
        h, i, d = self.hidden_size, self.intermediate_size, self.head_dim
        per_layer = (self.num_attention_heads + 2 * self.num_key_value_heads) * d * h \
            + self.num_attention_heads * d * h + 3 * i * h + 2 * h
        head = 0 if self.tie_word_embeddings else self.vocab_size * h
        return self.num_hidden_layers * per_layer + self.vocab_size * h + h + head
