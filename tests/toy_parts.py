"""Toy parts defined by the tests to show that another mixer, feed-forward or
position encoding can be registered, built and stepped without touching the
package: a mixer with per-request state of fixed size (a running mean of the
request's hidden vectors), written in plain tensor code on top of the step
context, and an architecture that alternates it with attention layers, runs one
layer twice and lets one run read another run's cache."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from paged_llm_b200.config.model import ModelConfig
from paged_llm_b200.config.registry import ARCHITECTURES, register_architecture
from paged_llm_b200.parts import (MIXERS, FixedState, LayerSpec, Mixer, ModelSpec, PartSpec, ScheduleEntry,
                                  TensorSpec, register_mixer)


class RunningMeanMixer(Mixer):
    """state = (sum of h over the request so far, count); out[t] = W (sum_t / count_t)."""

    def __init__(self, weights, hidden_size: int):
        self.hidden_size = hidden_size
        self.name = weights["proj"]
        self.w = None

    def cache_requirement(self):
        return FixedState((self.hidden_size + 1,))

    def tensor_specs(self):
        return {self.name: TensorSpec((self.hidden_size, self.hidden_size))}

    def load(self, tensors):
        self.w = tensors[self.name]

    def forward(self, h, ctx, cache):
        out = torch.empty_like(h)
        cu = ctx.host.cu
        for s, slot in enumerate(ctx.host.state_slots):
            assert slot >= 0, "a request of a model with state must own a slot"
            rows = h[cu[s]:cu[s + 1]].float()
            state = cache.state[slot]
            sums = state[:-1] + rows.cumsum(0)
            counts = state[-1] + torch.arange(1, rows.shape[0] + 1, device=h.device, dtype=torch.float32)
            state[:-1] = sums[-1]
            state[-1] = counts[-1]
            out[cu[s]:cu[s + 1]] = (sums / counts[:, None]).to(h.dtype)
        return ctx.ops.linear(out.contiguous(), self.w)


if "toy_running_mean" not in MIXERS:
    register_mixer("toy_running_mean")(RunningMeanMixer)


@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    intermediate_size: int = 0
    num_heads: int = 0
    head_dim: int = 0

    @classmethod
    def from_hf_dict(cls, d, architecture="ToyForCausalLM"):
        return cls(architecture, d["vocab_size"], d["hidden_size"], d["num_hidden_layers"],
                   d.get("max_position_embeddings", 256), d.get("torch_dtype", "float32"),
                   d["intermediate_size"], d["num_heads"], d["head_dim"])

    def to_hf_dict(self):
        return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                "num_hidden_layers": self.num_hidden_layers, "max_position_embeddings": self.max_position_embeddings,
                "torch_dtype": self.torch_dtype, "intermediate_size": self.intermediate_size,
                "num_heads": self.num_heads, "head_dim": self.head_dim}


def toy_spec(cfg: ToyConfig) -> ModelSpec:
    """Layers alternate running-mean and attention mixers; the schedule runs layer 1
    (attention) a second time at the end, reading the cache of its first run."""
    h = cfg.hidden_size
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"toy.layers.{i}."
        if i % 2 == 0:
            mixer = PartSpec("toy_running_mean", dict(hidden_size=h), {"proj": p + "mix.proj.weight"})
        else:
            mixer = PartSpec("paged_attention", dict(hidden_size=h, num_heads=cfg.num_heads, num_kv_heads=1,
                                                     head_dim=cfg.head_dim, position="rotary"),
                             {k: f"{p}attn.{k}.weight" for k in ("q_proj", "k_proj", "v_proj", "o_proj")})
        ffn = PartSpec("gated_mlp", dict(hidden_size=h, intermediate_size=cfg.intermediate_size),
                       {k: f"{p}ffn.{k}.weight" for k in ("gate_proj", "up_proj", "down_proj")})
        norms = {"input": PartSpec("rms_norm", dict(dim=h, eps=1e-5), {"weight": p + "norm1.weight"}),
                 "post_mixer": PartSpec("rms_norm", dict(dim=h, eps=1e-5), {"weight": p + "norm2.weight"})}
        layers.append(LayerSpec("pre_norm", mixer, ffn, norms))
    schedule = [ScheduleEntry(i) for i in range(cfg.num_hidden_layers)] + [ScheduleEntry(1, cache_from=1)]
    return ModelSpec(
        hidden_size=h, vocab_size=cfg.vocab_size,
        embedding=PartSpec("embedding", dict(vocab_size=cfg.vocab_size, hidden_size=h), {"weight": "toy.embed.weight"}),
        layers=layers, schedule=schedule,
        final_norm=PartSpec("rms_norm", dict(dim=h, eps=1e-5), {"weight": "toy.norm.weight"}),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, hidden_size=h, tied_to="toy.embed.weight"),
                      {"weight": "toy.head.weight"}),
        positions={"rotary": PartSpec("rotary", dict(head_dim=cfg.head_dim, theta=100.0))})


if "ToyForCausalLM" not in ARCHITECTURES:
    register_architecture("ToyForCausalLM", ToyConfig, toy_spec)

TOY = {"architectures": ["ToyForCausalLM"], "vocab_size": 61, "hidden_size": 48, "num_hidden_layers": 3,
       "intermediate_size": 40, "num_heads": 3, "head_dim": 16, "max_position_embeddings": 256,
       "torch_dtype": "float32"}


def plain_toy_logits(cfg: dict, w: dict, tokens) -> torch.Tensor:
    """Whole-sequence float32 oracle of the toy architecture, from tests/plain_llama.py's parts."""
    from tests import plain_llama as pl

    w = {k: v.float() for k, v in w.items()}
    h, heads, d = cfg["hidden_size"], cfg["num_heads"], cfg["head_dim"]
    toks = torch.as_tensor(tokens, dtype=torch.long)
    T = toks.numel()
    x = w["toy.embed.weight"][toks]
    cos, sin = pl.rotary_cos_sin(torch.arange(T), pl.inv_frequencies(d, 100.0, None))

    def layer(x, i, shared_kv=None):
        p = f"toy.layers.{i}."
        y = pl.rms_norm(x, w[p + "norm1.weight"], 1e-5)
        kv = None
        if i % 2 == 0:
            mean = y.cumsum(0) / torch.arange(1, T + 1)[:, None]
            a = mean @ w[p + "mix.proj.weight"].T
        else:
            q = pl.apply_rotary((y @ w[p + "attn.q_proj.weight"].T).view(T, heads, d), cos, sin)
            if shared_kv is None:
                k = pl.apply_rotary((y @ w[p + "attn.k_proj.weight"].T).view(T, 1, d), cos, sin)
                v = (y @ w[p + "attn.v_proj.weight"].T).view(T, 1, d)
                kv = (k, v)
            else:
                k, v = shared_kv
            a = pl.causal_attention(q, k, v, d ** -0.5).reshape(T, -1) @ w[p + "attn.o_proj.weight"].T
        x = x + a
        y = pl.rms_norm(x, w[p + "norm2.weight"], 1e-5)
        x = x + pl.gated_mlp(y, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"], w[p + "ffn.down_proj.weight"])
        return x, kv

    kv1 = None
    for i in range(cfg["num_hidden_layers"]):
        x, kv = layer(x, i)
        if i == 1:
            kv1 = kv
    x, _ = layer(x, 1, shared_kv=kv1)
    return pl.rms_norm(x, w["toy.norm.weight"], 1e-5) @ w["toy.embed.weight"].T
