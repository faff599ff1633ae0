"""Rotary position encoding.

inv_freq[j] = 1 / theta^(2j/d) in float32 (reference: pagedllm/model/llama.py:104),
optionally rescaled by the llama3 rule (llama.py:86-97); the angle of position p
is p * inv_freq[j] in float32 and the table holds its cosine and sine
(llama.py:111-115).  The rotation itself pairs element i with i + d/2
("half", llama.py:117-128) or 2i with 2i+1 ("interleaved", not used by Llama),
over the first `rotary_dim` elements of a head.

Frequencies are computed on the host in float32 with the reference's order of
operations, so that angles agree with it to rounding; the table is filled on
the device by a kernel of this package.
"""

from __future__ import annotations

import math

import torch

from .base import PositionEncoding, register_position_encoding


def llama3_rescale(inv_freq: torch.Tensor, factor: float, low_freq_factor: float,
                   high_freq_factor: float, original_max_position_embeddings: int) -> torch.Tensor:
    """Long wavelengths are divided by `factor`, short ones kept, and the band
    between blends the two linearly in 1/wavelength (llama.py:86-97)."""
    old_len = original_max_position_embeddings
    wavelen = 2 * math.pi / inv_freq
    long_wl, short_wl = old_len / low_freq_factor, old_len / high_freq_factor
    blend = (old_len / wavelen - low_freq_factor) / (high_freq_factor - low_freq_factor)
    out = torch.where(wavelen > long_wl, inv_freq / factor, inv_freq)
    band = (wavelen <= long_wl) & (wavelen >= short_wl)
    return torch.where(band, (1 - blend) * inv_freq / factor + blend * inv_freq, out)


@register_position_encoding("rotary")
class RotaryEncoding(PositionEncoding):
    def __init__(self, weights: dict[str, str], head_dim: int, theta: float,
                 scaling: dict | None = None, rotary_dim: int | None = None, pairing: str = "half"):
        self.head_dim = head_dim
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= head_dim:
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and within head_dim={head_dim}")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"unknown rotary pairing {pairing!r}")
        self.theta, self.scaling, self.pairing = float(theta), scaling, pairing
        self.table = None            # [P, rotary_dim/2, 2] float32: (cos, sin)
        self.max_positions = 0

    def inv_freq(self) -> torch.Tensor:
        rd = self.rotary_dim
        inv = 1.0 / (self.theta ** (torch.arange(0, rd, 2, dtype=torch.float32) / rd))
        if self.scaling:
            kind = self.scaling.get("rope_type", self.scaling.get("type"))
            if kind == "llama3":
                inv = llama3_rescale(inv, **{k: v for k, v in self.scaling.items() if k not in ("rope_type", "type")})
            elif kind not in (None, "default"):
                raise NotImplementedError(f"rope_type={kind!r} not supported (default and llama3 only)")
        return inv

    def prepare(self, max_positions, device, ops):
        self.max_positions = int(max_positions)
        self.table = ops.rope_table(self.inv_freq().to(device), self.max_positions)
