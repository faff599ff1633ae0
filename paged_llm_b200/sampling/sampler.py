"""Sampling from float32 logits: greedy, temperature, top-k, top-p.

Semantics follow the reference (pagedllm/sampler.py:10-35): temperature below
1e-5 means argmax; otherwise logits / temperature, keep the `top_k` largest,
keep a token while the probability mass of the tokens above it is <= `top_p`
(the largest always stays), softmax over what is left, one draw.

What differs: the draw uses a counter-based random stream per request (its
seed, the position it samples for), not one engine-wide generator
(pagedllm/engine.py:60), so a request's tokens do not depend on which other
requests share the step.  The draw is the Gumbel-max form of sampling from the
softmax: argmax(logit/T + g), g = -log(-log u).  All of it runs in kernels of
this package, one thread block per row.
"""

from __future__ import annotations

import numpy as np
import torch

MASK64 = (1 << 64) - 1


def request_seed(engine_seed: int, seq) -> int:
    """The 64-bit stream key of a request."""
    sp = seq.sampling_params
    if sp.seed is not None:
        return int(sp.seed) & MASK64
    x = (engine_seed * 0x9E3779B97F4A7C15 + (seq.seq_id + 1) * 0xD1B54A32D192ED03) & MASK64
    return x


class Sampler:
    def __init__(self, ops, seed: int = 0):
        self.ops = ops
        self.seed = int(seed)

    def sample(self, logits: torch.Tensor, seqs: list) -> list[int]:
        """logits: [n, vocab] float32 on the device; seqs: the n requests, whose
        `sampling_params` decide how each row is drawn.  Returns n token ids."""
        return self.sample_on_device(logits, seqs).tolist()

    def sample_on_device(self, logits: torch.Tensor, seqs: list) -> torch.Tensor:
        """The same, but the n token ids stay on the device (int32) and nothing waits."""
        n = logits.shape[0]
        assert n == len(seqs)
        params = [s.sampling_params for s in seqs]
        if all(p.greedy for p in params):
            return self.ops.argmax(logits)
        temps = np.array([p.temperature for p in params], np.float32)
        top_k = np.array([p.top_k if p.top_k > 0 else 0 for p in params], np.int32)
        top_p = np.array([p.top_p for p in params], np.float32)
        seeds = np.array([request_seed(self.seed, s) for s in seqs], np.uint64)
        counters = np.array([s.num_tokens for s in seqs], np.uint64)
        return self.ops.sample(logits, temps, top_k, top_p, seeds, counters)
