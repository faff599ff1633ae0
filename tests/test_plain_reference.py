"""The plain implementation: held to the reference's own model code through the
stored outputs of tests/golden/, and its parts checked against independent
formulations."""

import math
import os

import numpy as np
import pytest
import torch

from tests import plain_llama
from tests.tiny import TINIES, make_folder, read_folder

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "reference_logits.npz")


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_plain_equals_the_reference_model(tmp_path, name):
    gold = np.load(GOLDEN)
    hf, init = TINIES[name]
    make_folder(tmp_path, hf, init)
    cfg, w = read_folder(tmp_path)
    got = plain_llama.forward_logits(cfg, w, gold[f"{name}_tokens"].tolist()).numpy()
    np.testing.assert_allclose(got, gold[f"{name}_logits"], atol=2e-5, rtol=1e-5)


def test_float64_agrees_with_float32(tmp_path):
    hf, init = TINIES["B"]
    make_folder(tmp_path, hf, init)
    cfg, w = read_folder(tmp_path)
    toks = list(range(1, 60))
    a = plain_llama.forward_logits(cfg, w, toks)
    b = plain_llama.forward_logits(cfg, w, toks, dtype=torch.float64)
    assert float((a - b).abs().max()) < 5e-5


def test_attention_against_sdpa_and_window():
    g = torch.Generator().manual_seed(0)
    T, heads, kvh, d = 37, 6, 2, 16
    q, k, v = (torch.randn(T, h, d, generator=g) for h in (heads, kvh, kvh))
    got = plain_llama.causal_attention(q, k, v, d ** -0.5)
    kk, vv = k.repeat_interleave(3, 1), v.repeat_interleave(3, 1)
    want = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(0, 1), kk.transpose(0, 1), vv.transpose(0, 1), is_causal=True).transpose(0, 1)
    torch.testing.assert_close(got, want, atol=1e-5, rtol=1e-5)
    win = plain_llama.causal_attention(q, k, v, d ** -0.5, window=5)
    for t in (0, 4, 5, 20, 36):
        lo = max(0, t - 4)
        s = torch.einsum("hd,khd->hk", q[t], kk[lo:t + 1]) * d ** -0.5
        torch.testing.assert_close(win[t], torch.einsum("hk,khd->hd", s.softmax(-1), vv[lo:t + 1]), atol=1e-5, rtol=1e-5)


def test_rotary_is_a_rotation_by_relative_position():
    inv = plain_llama.inv_frequencies(32, 10000.0, None)
    g = torch.Generator().manual_seed(1)
    q, k = torch.randn(1, 1, 32, generator=g), torch.randn(1, 1, 32, generator=g)
    def dot(pq, pk):
        cq, sq = plain_llama.rotary_cos_sin(torch.tensor([pq]), inv)
        ck, sk = plain_llama.rotary_cos_sin(torch.tensor([pk]), inv)
        return float((plain_llama.apply_rotary(q, cq, sq) * plain_llama.apply_rotary(k, ck, sk)).sum())
    assert abs(dot(7, 3) - dot(104, 100)) < 1e-3 and abs(dot(7, 3) - dot(7, 4)) > 1e-4
    assert abs(float(plain_llama.apply_rotary(q, *plain_llama.rotary_cos_sin(torch.tensor([9]), inv)).norm()
                     - q.norm())) < 1e-5


def test_llama3_scaling_bands():
    s = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
         "original_max_position_embeddings": 64}
    base = plain_llama.inv_frequencies(32, 500000.0, None)
    scaled = plain_llama.inv_frequencies(32, 500000.0, s)
    wavelen = 2 * math.pi / base
    assert torch.equal(scaled[wavelen < 16], base[wavelen < 16])                 # short waves untouched
    torch.testing.assert_close(scaled[wavelen > 64], base[wavelen > 64] / 8)     # long waves divided
    mid = (wavelen >= 16) & (wavelen <= 64)
    assert mid.any() and ((scaled[mid] <= base[mid]) & (scaled[mid] >= base[mid] / 8)).all()


def test_rms_norm_and_mlp():
    x = torch.tensor([[3.0, 4.0]])
    torch.testing.assert_close(plain_llama.rms_norm(x, torch.tensor([1.0, 2.0]), 0.0),
                               torch.tensor([[3.0, 8.0]]) / math.sqrt(12.5))
    g = torch.Generator().manual_seed(2)
    x, wg, wu, wd = (torch.randn(*s, generator=g) for s in ((5, 8), (12, 8), (12, 8), (8, 12)))
    want = (torch.nn.functional.silu(x @ wg.T) * (x @ wu.T)) @ wd.T
    torch.testing.assert_close(plain_llama.gated_mlp(x, wg, wu, wd), want)


def test_sampling_filter():
    logits = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0])
    p = plain_llama.sampling_distribution(logits, 1.0, top_k=2)
    assert (p[2:] == 0).all() and abs(float(p.sum()) - 1) < 1e-6
    full = logits.softmax(-1)
    p = plain_llama.sampling_distribution(logits, 1.0, top_p=float(full[0]) + 1e-3)
    assert (p > 0).tolist() == [True, True, False, False, False]    # kept while the mass above is <= top_p
    p = plain_llama.sampling_distribution(logits, 1.0, top_p=1e-6)
    assert (p > 0).tolist() == [True, False, False, False, False]   # the largest always stays
