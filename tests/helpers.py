"""Shared helpers of the GPU tests."""

from __future__ import annotations

import numpy as np
import torch

from tests import plain_llama
from tests.tiny import TINIES, make_folder, random_tokens, read_folder

# Tolerances (never widened to make a test pass):
#  float32: the engine and the plain implementation differ by summation order only.
#  bfloat16: activations are rounded to 8 bits of mantissa between kernels; the
#  bound is relative to the largest logit of the model.
#  bfloat16 against the float32 engine on the same weight values: only the rounding of
#  activations is left, which is what a misplaced key or a stale page would have to hide in.
F32_TOL = 2e-5
BF16_REL_TOL = 3e-2
#  Measured on a B200 over every schedule of the tiny and the wide models: at most 1.5e-2 of the largest
#  logit (the far tail of some 10^5 logits per comparison).
BF16_VS_F32_TOL = 2e-2


def model_folder(tmp_path_factory, name: str, dtype: str = "float32"):
    hf, init = TINIES[name]
    d = tmp_path_factory.mktemp(f"tiny{name}_{dtype}")
    make_folder(d, hf, init, dtype=dtype)
    return str(d)


def plain_logits(folder: str, tokens) -> np.ndarray:
    cfg, w = read_folder(folder)
    return plain_llama.forward_logits(cfg, w, tokens).numpy()


def assert_logits_close(got: np.ndarray, want: np.ndarray, dtype: str, what: str = ""):
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert np.isfinite(got).all(), f"{what}: non-finite logits"
    err = np.abs(got - want)
    if dtype == "float32":
        tol = F32_TOL * max(1.0, float(np.abs(want).max()))
    else:
        tol = BF16_REL_TOL * float(np.abs(want).max())
    worst = np.unravel_index(err.argmax(), err.shape)
    assert err.max() <= tol, (f"{what}: max |diff| {err.max():.3e} > {tol:.3e} at position {worst[0]}, "
                              f"token {worst[1]}; first bad position {int(np.argmax(err.max(axis=1) > tol))}")


# (what, largest difference / largest logit) of every bfloat16-against-float32 comparison of the run;
# tests/conftest.py prints the largest at the end, so that the tolerance can be held against it.
BF16_VS_F32_SEEN: list[tuple[str, float]] = []


def assert_bf16_close_to_f32(got: np.ndarray, f32: np.ndarray, what: str = "") -> float:
    """The bfloat16 engine's logits against the float32 engine's for the same trace."""
    assert got.shape == f32.shape, f"{what}: shape {got.shape} != {f32.shape}"
    assert np.isfinite(got).all() and np.isfinite(f32).all(), f"{what}: non-finite logits"
    err = np.abs(got - f32)
    tol = BF16_VS_F32_TOL * float(np.abs(f32).max())
    BF16_VS_F32_SEEN.append((what, float(err.max() / max(np.abs(f32).max(), 1e-30))))
    worst = np.unravel_index(err.argmax(), err.shape)
    assert err.max() <= tol, (f"{what}: max |diff| {err.max():.3e} > {tol:.3e} at row {worst[0]}, token {worst[1]}; "
                              f"first bad row {int(np.argmax(err.max(axis=1) > tol))}")
    return float(err.max() / max(np.abs(f32).max(), 1e-30))


def requests_for(vocab: int, lengths, seed: int = 0) -> dict[str, list[int]]:
    return {f"r{i}": random_tokens(vocab, n, seed * 100 + i) for i, n in enumerate(lengths)}
