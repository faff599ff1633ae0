"""Plain version of the sampler's draw, for tests: the counter-based random
stream and the Gumbel-max draw over the filtered logits, in numpy.

The filter is the reference's (pagedllm/sampler.py:17-29, restated in
tests/plain_llama.py:filter_logits); the stream is this package's own: uniform
u(seed, counter, i) from a splitmix64 mix, g = -log(-log u), token =
argmax(logit / T + g) over the kept tokens.
"""

from __future__ import annotations

import numpy as np
import torch

from tests.plain_llama import filter_logits

M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def uniforms(seed: int, counter: int, n: int) -> np.ndarray:
    """u_i in (0, 1), i = 0..n-1, float32."""
    with np.errstate(over="ignore"):
        i = np.arange(n, dtype=np.uint64)
        x = np.uint64(seed) + np.uint64(counter) * np.uint64(0x9E3779B97F4A7C15) + i * np.uint64(0xBF58476D1CE4E5B9)
        x ^= x >> np.uint64(30)
        x *= np.uint64(0xBF58476D1CE4E5B9)
        x ^= x >> np.uint64(27)
        x *= np.uint64(0x94D049BB133111EB)
        x ^= x >> np.uint64(31)
    return (((x >> np.uint64(40)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)).astype(np.float32)


def gumbel_scores(row: np.ndarray, temperature: float, top_k: int, top_p: float, seed: int, counter: int) -> np.ndarray:
    kept = filter_logits(torch.from_numpy(row.astype(np.float32)), float(temperature), int(top_k), float(top_p)).numpy()
    u = uniforms(seed, counter, row.size)
    g = -np.log(-np.log(u.astype(np.float64))).astype(np.float32)
    return kept + g


def sample_rows(logits: np.ndarray, temps, top_k, top_p, seeds, counters) -> list[int]:
    out = []
    for r in range(logits.shape[0]):
        if temps[r] < 1e-5:
            out.append(int(logits[r].argmax()))
        else:
            out.append(int(gumbel_scores(logits[r], temps[r], top_k[r], top_p[r], int(seeds[r]), int(counters[r])).argmax()))
    return out
