"""Per-request sampling options, as in the reference (pagedllm/sequence.py:9-20).

`seed` is an addition: when set, the request draws from its own counter-based
random stream (seed, position), so what it samples does not depend on which
other requests share its steps.  When None the engine derives the stream from
its own seed and the request's id.
"""

from __future__ import annotations

from dataclasses import dataclass

GREEDY_EPS = 1e-5


@dataclass
class SamplingParams:
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1                 # <= 0: off
    max_tokens: int = 128
    ignore_eos: bool = False
    stop_token_ids: tuple[int, ...] = ()
    seed: int | None = None

    def __post_init__(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be >= 1")
        self.stop_token_ids = tuple(self.stop_token_ids)

    @property
    def greedy(self) -> bool:
        return self.temperature < GREEDY_EPS
