"""Plain, slow implementation of the Llama dense decoder, for tests only.

Whole sequences, no cache, no batching, one function for each part, float32 (or
float64) on the CPU.  It shares no code with the product package: it imports
nothing from it and takes plain dicts (the config.json dict and a dict of
tensors under their HuggingFace names).

Every function is written from the formulas of the reference implementation
(xiyiji/paged-llm); the file:line citations point into that project.  The
comparison of this file with the reference's own model code, run once on the
CPU, is stored under tests/golden/ (see tests/golden/make_golden.py).
"""

from __future__ import annotations

import math

import torch


# --------------------------------------------------------------------------- config

def read_config(cfg: dict) -> dict:
    """Resolve defaults the way pagedllm/model/llama.py:37-60 does.

    rope parameters: `rope_parameters` first, else `rope_scaling`; theta from the
    dict, else the top-level key, else 10000.0; a rope type of "default" (or no
    type) means no scaling (llama.py:42-45).
    """
    heads = cfg["num_attention_heads"]
    rope = dict(cfg.get("rope_parameters") or cfg.get("rope_scaling") or {})
    theta = rope.pop("rope_theta", None) or cfg.get("rope_theta", 10000.0)
    rope_type = rope.get("rope_type", rope.get("type", "default"))
    return {
        "vocab": cfg["vocab_size"],
        "hidden": cfg["hidden_size"],
        "inter": cfg["intermediate_size"],
        "layers": cfg["num_hidden_layers"],
        "heads": heads,
        "kv_heads": cfg.get("num_key_value_heads", heads),
        "head_dim": cfg.get("head_dim") or cfg["hidden_size"] // heads,
        "eps": cfg.get("rms_norm_eps", 1e-5),
        "theta": float(theta),
        "scaling": rope if rope_type != "default" else None,
        "tied": cfg.get("tie_word_embeddings", False),
    }


# --------------------------------------------------------------------------- parts

def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w, eps inside the root (llama.py:80-83)."""
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * weight


def inv_frequencies(head_dim: int, theta: float, scaling: dict | None) -> torch.Tensor:
    """inv_freq[j] = 1 / theta^(2j/d) in float32 (llama.py:104), then the optional
    llama3 rescale (llama.py:86-97).  Kept in float32 on purpose: the reference
    builds its table in float32 and the angles must agree to rounding."""
    exponents = torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim
    inv_freq = 1.0 / (theta ** exponents)
    if scaling is None:
        return inv_freq
    kind = scaling.get("rope_type", scaling.get("type"))
    if kind != "llama3":
        raise NotImplementedError(kind)               # llama.py:109-110
    factor = scaling["factor"]
    low = scaling.get("low_freq_factor", 1.0)
    high = scaling.get("high_freq_factor", 4.0)
    old_len = scaling.get("original_max_position_embeddings", 8192)
    wavelen = 2 * math.pi / inv_freq
    smooth = (old_len / wavelen - low) / (high - low)
    out = torch.where(wavelen > old_len / low, inv_freq / factor, inv_freq)
    middle = (wavelen <= old_len / low) & (wavelen >= old_len / high)
    blended = (1 - smooth) * inv_freq / factor + smooth * inv_freq
    return torch.where(middle, blended, out)


def rotary_cos_sin(positions: torch.Tensor, inv_freq: torch.Tensor):
    """angle[p, j] = p * inv_freq[j] in float32; the half table is repeated twice
    along the last axis (llama.py:111-115)."""
    ang = torch.outer(positions.to(torch.float32), inv_freq)
    ang = torch.cat([ang, ang], dim=-1)
    return ang.cos(), ang.sin()


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: [T, heads, d].  Element i pairs with i + d/2 (rotate-half, llama.py:117-128)."""
    half = x.shape[-1] // 2
    rotated = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos[:, None, :].to(x.dtype) + rotated * sin[:, None, :].to(x.dtype)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                     window: int | None = None, softcap: float | None = None, slopes=None) -> torch.Tensor:
    """q: [T, heads, d], k/v: [T, kv_heads, d], one whole sequence.

    Query head h reads kv head h // (heads // kv_heads); scores scaled, keys after
    the query's position masked out, softmax over keys, weighted sum of values
    (pagedllm/attention/reference.py:23-55).  `window`, which the reference does
    not have, keeps only the last `window` keys (the query's own included); `softcap` c turns a scaled score s into c * tanh(s / c) and
    `slopes` (one number per query head) adds slope * (key position - query position): two
    score modifiers of this engine's attention part, neither of which the reference has.
    """
    T, heads, _ = q.shape
    group = heads // k.shape[1]
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    scores = torch.einsum("qhd,khd->hqk", q, k) * scale
    pos = torch.arange(T)
    if softcap:
        scores = softcap * torch.tanh(scores / softcap)
    if slopes is not None:
        scores = scores + torch.as_tensor(slopes, dtype=scores.dtype)[:, None, None] * (pos[None, None, :] - pos[None, :, None])
    hidden = pos[None, :] > pos[:, None]
    if window is not None:
        hidden = hidden | (pos[None, :] <= pos[:, None] - window)
    scores = scores.masked_fill(hidden[None], float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    return torch.einsum("hqk,khd->qhd", probs, v)


def gated_mlp(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """down(silu(gate(x)) * up(x)), no bias (llama.py:163-171)."""
    g = x @ w_gate.T
    u = x @ w_up.T
    return (g * torch.sigmoid(g) * u) @ w_down.T


def attention_block(x, w, prefix, c, cos, sin, window=None):
    """Projections, rotary on q and k, attention, output projection (llama.py:146-160)."""
    T = x.shape[0]
    q = (x @ w[prefix + "q_proj.weight"].T).view(T, c["heads"], c["head_dim"])
    k = (x @ w[prefix + "k_proj.weight"].T).view(T, c["kv_heads"], c["head_dim"])
    v = (x @ w[prefix + "v_proj.weight"].T).view(T, c["kv_heads"], c["head_dim"])
    q = apply_rotary(q, cos, sin)
    k = apply_rotary(k, cos, sin)
    o = causal_attention(q, k, v, c["head_dim"] ** -0.5, window)     # scale: llama.py:138
    return o.reshape(T, -1) @ w[prefix + "o_proj.weight"].T


def decoder_layer(x, w, i, c, cos, sin):
    """Pre-norm block with two residual sums (llama.py:182-185)."""
    p = f"model.layers.{i}."
    h = rms_norm(x, w[p + "input_layernorm.weight"], c["eps"])
    x = x + attention_block(h, w, p + "self_attn.", c, cos, sin)
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"])
    x = x + gated_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return x


# --------------------------------------------------------------------------- whole model

def forward_logits(cfg: dict, weights: dict, tokens, dtype=torch.float32, rows=None) -> torch.Tensor:
    """Logits [T, vocab] at every position of one whole sequence (llama.py:196-216).

    `weights` holds tensors under HuggingFace names; they are used in `dtype`
    (float32 or float64) whatever they are stored in.  `rows`: the positions whose
    logits are wanted (the head is then applied to those rows only, which the
    reference does too: llama.py:214-216); None means all of them.
    """
    c = read_config(cfg)
    w = {k: t.to(dtype) for k, t in weights.items()}
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["model.embed_tokens.weight"][tokens]
    inv_freq = inv_frequencies(c["head_dim"], c["theta"], c["scaling"])
    cos, sin = rotary_cos_sin(torch.arange(tokens.numel()), inv_freq)
    for i in range(c["layers"]):
        x = decoder_layer(x, w, i, c, cos, sin)
    if rows is not None:
        x = x[torch.as_tensor(rows, dtype=torch.long)]
    x = rms_norm(x, w["model.norm.weight"], c["eps"])
    head = w["model.embed_tokens.weight"] if c["tied"] and "lm_head.weight" not in w else w["lm_head.weight"]
    return (x @ head.T).to(torch.float32)


def greedy_generate(cfg: dict, weights: dict, prompt, max_tokens: int) -> list[int]:
    """Greedy continuation, recomputing the whole sequence for every token."""
    toks = list(prompt)
    for _ in range(max_tokens):
        toks.append(int(forward_logits(cfg, weights, toks)[-1].argmax()))
    return toks[len(prompt):]


# --------------------------------------------------------------------------- sampling

def filter_logits(logits: torch.Tensor, temperature: float, top_k: int, top_p: float) -> torch.Tensor:
    """One row: temperature, then keep rank < top_k and exclusive cumulative
    probability <= top_p over the descending order; the rest becomes -inf
    (pagedllm/sampler.py:17-29)."""
    logits = logits / max(temperature, 1e-5)
    vocab = logits.numel()
    k = top_k if top_k > 0 else vocab
    if k < vocab or top_p < 1.0:
        srt, idx = logits.sort(descending=True)
        probs = srt.softmax(-1)
        before = probs.cumsum(-1) - probs
        drop = (torch.arange(vocab) >= k) | (before > top_p)
        srt = srt.masked_fill(drop, float("-inf"))
        logits = torch.full_like(logits, float("-inf")).scatter(-1, idx, srt)
    return logits


def sampling_distribution(logits: torch.Tensor, temperature: float, top_k: int = -1, top_p: float = 1.0) -> torch.Tensor:
    """Probabilities the sampler draws from (sampler.py:30)."""
    return filter_logits(logits.float(), temperature, top_k, top_p).softmax(-1)
