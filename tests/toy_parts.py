"""Toy parts defined by the tests to show that another mixer, feed-forward or
position encoding can be registered, built and stepped without touching the
package: a mixer with per-request state of fixed size (a running mean of the
request's hidden vectors), written in plain tensor code on top of the step
context, and an architecture that alternates it with attention layers, runs one
layer twice and lets one run read another run's cache; and a second architecture
with a learned table of absolute positions that its embedding adds (attention
then rotates nothing), a feed-forward that routes each token to some of its
experts, and a head of its own."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from paged_llm_b200.config.model import ModelConfig
from paged_llm_b200.config.registry import ARCHITECTURES, register_architecture
from paged_llm_b200.parts import (EMBEDDINGS, FEED_FORWARDS, MIXERS, POSITION_ENCODINGS, Embedding, FeedForward,
                                  FixedState, LayerSpec, Mixer, ModelSpec, PartSpec, PositionEncoding, ScheduleEntry,
                                  TensorSpec, materialize, register_embedding, register_feed_forward, register_mixer,
                                  register_position_encoding)


class RunningMeanMixer(Mixer):
    """state = (sum of h over the request so far, count); out[t] = W (sum_t / count_t)."""

    capturable = False          # walks the requests on the host

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


class DeviceRunningMeanMixer(Mixer):
    """The same running mean, written so that a step can be captured and replayed: it reads the
    step's metadata on the device only (request of each token, first row of each request, state
    slots, positions) and launches a fixed sequence of tensor operations whatever the batch holds.
    state = sum of h over the request so far; the count is the token's position + 1.  Rows and
    requests that pad a captured batch (request -1, slot -1) add nothing."""

    capturable = True

    def __init__(self, weights, hidden_size: int):
        self.hidden_size = hidden_size
        self.name = weights["proj"]
        self.w = None

    def cache_requirement(self):
        return FixedState((self.hidden_size,))

    def tensor_specs(self):
        return {self.name: TensorSpec((self.hidden_size, self.hidden_size))}

    def load(self, tensors):
        self.w = tensors[self.name]

    def forward(self, h, ctx, cache):
        seq = ctx.token_seq.long()                             # [T], -1 for padding rows
        real = seq >= 0
        seq = seq.clamp(min=0)
        cu = ctx.cu_seqlens_q.long()                           # [S + 1]
        slots = ctx.state_slots.long()                         # [S], -1 for padding requests
        owned = slots >= 0
        slots = slots.clamp(min=0)
        state = cache.state
        csum = (h.float() * real[:, None]).cumsum(0)           # over all rows of the step
        first = cu[seq]                                        # first row of the token's request
        before = torch.where((first > 0)[:, None], csum[(first - 1).clamp(min=0)], torch.zeros_like(csum))
        run = csum - before + state[slots[seq]]                # the request's sum up to and including the token
        out = (run / (ctx.positions.float() + 1)[:, None]).to(h.dtype)
        last = (cu[1:] - 1).clamp(min=0)
        grew = owned & (cu[1:] > cu[:-1])
        state.index_add_(0, slots, torch.where(grew[:, None], run[last] - state[slots], torch.zeros_like(run[last])))
        return ctx.ops.linear(out.contiguous(), self.w)


if "toy_running_mean_device" not in MIXERS:
    register_mixer("toy_running_mean_device")(DeviceRunningMeanMixer)


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


def toy_spec(cfg: ToyConfig, mean_mixer: str = "toy_running_mean") -> ModelSpec:
    """Layers alternate running-mean and attention mixers; the schedule runs layer 1
    (attention) a second time at the end, reading the cache of its first run."""
    h = cfg.hidden_size
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"toy.layers.{i}."
        if i % 2 == 0:
            mixer = PartSpec(mean_mixer, dict(hidden_size=h), {"proj": p + "mix.proj.weight"})
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
if "DeviceToyForCausalLM" not in ARCHITECTURES:       # the same model with the capturable running mean
    register_architecture("DeviceToyForCausalLM", ToyConfig,
                          lambda cfg: toy_spec(cfg, mean_mixer="toy_running_mean_device"))

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


# --------------------------------------------------------------------------- a second toy: learned positions, routing

class LearnedAbsolutePositions(PositionEncoding):
    """A table with one vector of the model's width per position, read from the checkpoint."""

    capturable = False          # `encode` checks the step's positions on the host

    def __init__(self, weights, max_positions: int, hidden_size: int):
        self.rows, self.hidden_size = max_positions, hidden_size
        self.name = weights["table"]
        self.table = None

    def tensor_specs(self):
        return {self.name: TensorSpec((self.rows, self.hidden_size))}

    def load(self, tensors):
        self.table = tensors[self.name].contiguous()

    def prepare(self, max_positions, device, ops):
        pass        # nothing to compute: the table is a weight; `encode` refuses positions beyond it

    def encode(self, ctx):
        """[T, hidden] float32: the vectors of the step's positions."""
        if max(ctx.host.k_lens) > self.rows:
            raise ValueError(f"a request reaches position {max(ctx.host.k_lens) - 1}, the table has {self.rows} rows")
        return ctx.ops.embedding(self.table, ctx.positions)


class PositionedEmbedding(Embedding):
    """x[t] = E[ids[t]] + P[position[t]], summed in float32."""

    def __init__(self, weights, vocab_size: int, hidden_size: int, position):
        self.vocab_size, self.hidden_size, self.position = vocab_size, hidden_size, position
        self.name = weights["weight"]
        self.weight = None

    def tensor_specs(self):
        return {self.name: TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors):
        self.weight = tensors[self.name].contiguous()

    def forward(self, ids, ctx):
        return ctx.ops.embedding(self.weight, ids).add_(self.position.encode(ctx))


class RoutedMLP(FeedForward):
    """Router logits in float32, the `top_k` largest kept and softmaxed over the kept ones;
    out[t] = sum over kept experts e of p[t, e] * down_e(silu(gate_e h[t]) * up_e h[t])."""

    capturable = False          # counts each expert's rows on the host

    def __init__(self, weights, hidden_size: int, intermediate_size: int, num_experts: int, top_k: int):
        if not 0 < top_k <= num_experts:
            raise ValueError(f"top_k={top_k} must lie in 1..num_experts={num_experts}")
        self.h, self.i, self.e, self.k = hidden_size, intermediate_size, num_experts, top_k
        self.names = weights
        self.router = self.gate_up = self.down = None

    def _expert(self, e, which):
        return self.names["experts"].format(expert=e, proj=which)

    def tensor_specs(self):
        out = {self.names["router"]: TensorSpec((self.e, self.h))}
        for e in range(self.e):
            out[self._expert(e, "gate_proj")] = TensorSpec((self.i, self.h))
            out[self._expert(e, "up_proj")] = TensorSpec((self.i, self.h))
            out[self._expert(e, "down_proj")] = TensorSpec((self.h, self.i))
        return out

    def load(self, tensors):
        self.router = tensors[self.names["router"]].float()
        self.gate_up = [torch.cat([tensors[self._expert(e, "gate_proj")], tensors[self._expert(e, "up_proj")]]).contiguous()
                        for e in range(self.e)]
        self.down = [tensors[self._expert(e, "down_proj")].contiguous() for e in range(self.e)]

    def forward(self, h, ctx):
        ops = ctx.ops
        logits = h.float() @ self.router.T
        top, chosen = logits.topk(self.k, dim=-1)
        probs = torch.softmax(top, dim=-1)
        out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
        for e in range(self.e):
            rows, slot = (chosen == e).nonzero(as_tuple=True)
            if rows.numel() == 0:
                continue
            y = materialize(ops.linear(ops.gated_silu_linear(h[rows].contiguous(), self.gate_up[e]), self.down[e]), ops)
            out.index_add_(0, rows, y.float() * probs[rows, slot][:, None])
        return out.to(h.dtype)


if "toy_learned_absolute" not in POSITION_ENCODINGS:
    register_position_encoding("toy_learned_absolute")(LearnedAbsolutePositions)
if "toy_positioned_embedding" not in EMBEDDINGS:
    register_embedding("toy_positioned_embedding")(PositionedEmbedding)
if "toy_routed_mlp" not in FEED_FORWARDS:
    register_feed_forward("toy_routed_mlp")(RoutedMLP)


@dataclass(frozen=True)
class RoutedToyConfig(ModelConfig):
    intermediate_size: int = 0
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    num_experts: int = 0
    top_k: int = 0
    eps: float = 1e-5

    KEYS = ("intermediate_size", "num_heads", "num_kv_heads", "head_dim", "num_experts", "top_k", "eps")

    @classmethod
    def from_hf_dict(cls, d, architecture="RoutedToyForCausalLM"):
        return cls(architecture, d["vocab_size"], d["hidden_size"], d["num_hidden_layers"],
                   d["max_position_embeddings"], d.get("torch_dtype", "float32"), *(d[k] for k in cls.KEYS))

    def to_hf_dict(self):
        return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "hidden_size": self.hidden_size,
                "num_hidden_layers": self.num_hidden_layers, "max_position_embeddings": self.max_position_embeddings,
                "torch_dtype": self.torch_dtype, **{k: getattr(self, k) for k in self.KEYS}}


def routed_toy_spec(cfg: RoutedToyConfig) -> ModelSpec:
    h = cfg.hidden_size
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"rt.layers.{i}."
        mixer = PartSpec("paged_attention", dict(hidden_size=h, num_heads=cfg.num_heads, num_kv_heads=cfg.num_kv_heads,
                                                 head_dim=cfg.head_dim, position=None),
                         {k: f"{p}attn.{k}.weight" for k in ("q_proj", "k_proj", "v_proj", "o_proj")})
        ffn = PartSpec("toy_routed_mlp", dict(hidden_size=h, intermediate_size=cfg.intermediate_size,
                                              num_experts=cfg.num_experts, top_k=cfg.top_k),
                       {"router": p + "router.weight", "experts": p + "experts.{expert}.{proj}.weight"})
        norms = {"input": PartSpec("rms_norm", dict(dim=h, eps=cfg.eps), {"weight": p + "norm1.weight"}),
                 "post_mixer": PartSpec("rms_norm", dict(dim=h, eps=cfg.eps), {"weight": p + "norm2.weight"})}
        layers.append(LayerSpec("pre_norm", mixer, ffn, norms))
    return ModelSpec(
        hidden_size=h, vocab_size=cfg.vocab_size,
        embedding=PartSpec("toy_positioned_embedding", dict(vocab_size=cfg.vocab_size, hidden_size=h, position="learned"),
                           {"weight": "rt.embed.weight"}),
        layers=layers, schedule=[ScheduleEntry(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rms_norm", dict(dim=h, eps=cfg.eps), {"weight": "rt.norm.weight"}),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, hidden_size=h), {"weight": "rt.head.weight"}),
        positions={"learned": PartSpec("toy_learned_absolute", dict(max_positions=cfg.max_position_embeddings,
                                                                    hidden_size=h), {"table": "rt.positions.weight"})})


if "RoutedToyForCausalLM" not in ARCHITECTURES:
    register_architecture("RoutedToyForCausalLM", RoutedToyConfig, routed_toy_spec)

# top_k < num_experts: a token's experts change with its hidden vector (float32 only: in bfloat16 a
# near-tie may fall to the other side, which is a property of routing, not a fault of the engine).
ROUTED_TOY_A = {"architectures": ["RoutedToyForCausalLM"], "vocab_size": 53, "hidden_size": 40, "num_hidden_layers": 2,
                "intermediate_size": 24, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16, "num_experts": 4,
                "top_k": 2, "eps": 1e-5, "max_position_embeddings": 160, "torch_dtype": "float32"}
# top_k == num_experts: every expert weighs in, so the output is continuous in the router's logits.
ROUTED_TOY_B = {"architectures": ["RoutedToyForCausalLM"], "vocab_size": 47, "hidden_size": 96, "num_hidden_layers": 3,
                "intermediate_size": 64, "num_heads": 3, "num_kv_heads": 1, "head_dim": 32, "num_experts": 3,
                "top_k": 3, "eps": 1e-6, "max_position_embeddings": 192, "torch_dtype": "float32"}


def plain_routed_toy_logits(cfg: dict, w: dict, tokens) -> torch.Tensor:
    """Whole-sequence float32 oracle of the routed toy, from tests/plain_llama.py's parts."""
    from tests import plain_llama as pl

    w = {k: v.float() for k, v in w.items()}
    heads, kvh, d = cfg["num_heads"], cfg["num_kv_heads"], cfg["head_dim"]
    toks = torch.as_tensor(tokens, dtype=torch.long)
    T = toks.numel()
    x = w["rt.embed.weight"][toks] + w["rt.positions.weight"][:T]
    for i in range(cfg["num_hidden_layers"]):
        p = f"rt.layers.{i}."
        y = pl.rms_norm(x, w[p + "norm1.weight"], cfg["eps"])
        q = (y @ w[p + "attn.q_proj.weight"].T).view(T, heads, d)
        k = (y @ w[p + "attn.k_proj.weight"].T).view(T, kvh, d)
        v = (y @ w[p + "attn.v_proj.weight"].T).view(T, kvh, d)
        x = x + pl.causal_attention(q, k, v, d ** -0.5).reshape(T, -1) @ w[p + "attn.o_proj.weight"].T
        y = pl.rms_norm(x, w[p + "norm2.weight"], cfg["eps"])
        top, chosen = (y @ w[p + "router.weight"].T).topk(cfg["top_k"], dim=-1)
        probs = torch.softmax(top, dim=-1)
        f = torch.zeros_like(x)
        for t in range(T):
            for j in range(cfg["top_k"]):
                e = f"{p}experts.{int(chosen[t, j])}."
                f[t] += probs[t, j] * pl.gated_mlp(y[t:t + 1], w[e + "gate_proj.weight"], w[e + "up_proj.weight"],
                                                   w[e + "down_proj.weight"])[0]
        x = x + f
    return pl.rms_norm(x, w["rt.norm.weight"], cfg["eps"]) @ w["rt.head.weight"].T


# --------------------------------------------------------------------------- a Llama with score modifiers

def biased_llama_case(folder, dtype: str = "float32"):
    """A Llama (the third tiny configuration) whose attention rotates nothing and instead adds,
    per head, a slope times the distance to the key, with a cap on the scores of its second
    layer: parameters of the attention part, chosen by a spec of the test's own.  Writes the
    model folder; returns (config dict, float32 weights, requests, plain logits function)."""
    from paged_llm_b200.config import LlamaConfig
    from paged_llm_b200.models.llama import llama_spec
    from paged_llm_b200.weights import write_model_folder
    from tests import plain_llama
    from tests.tiny import TINY_C, random_tokens, read_folder

    heads = TINY_C["num_attention_heads"]
    slopes = [2.0 ** -(1 + 6.0 * h / heads) for h in range(heads)]
    caps = (None, 0.8)

    def spec(cfg):
        s = llama_spec(cfg)
        for layer, cap in zip(s.layers, caps):
            layer.mixer.params.update(position=None, position_slopes=slopes, score_cap=cap)
        return s
    if "BiasedLlama" not in ARCHITECTURES:
        register_architecture("BiasedLlama", LlamaConfig, spec)
    cfg = LlamaConfig.from_hf_dict({**TINY_C, "architectures": ["BiasedLlama"]}, architecture="BiasedLlama")
    write_model_folder(str(folder), cfg, seed=8, std=0.15, dtype=dtype)
    hf, w = read_folder(folder)
    w = {k: v.float() for k, v in w.items()}
    c = plain_llama.read_config(hf)
    reqs = {"a": random_tokens(hf["vocab_size"], 90, 1), "b": random_tokens(hf["vocab_size"], 150, 2),
            "c": random_tokens(hf["vocab_size"], 33, 3)}

    def plain(toks):
        T = len(toks)
        x = w["model.embed_tokens.weight"][torch.tensor(toks)]
        for i, cap in enumerate(caps):
            p = f"model.layers.{i}."
            h = plain_llama.rms_norm(x, w[p + "input_layernorm.weight"], c["eps"])
            q = (h @ w[p + "self_attn.q_proj.weight"].T).view(T, c["heads"], c["head_dim"])
            k = (h @ w[p + "self_attn.k_proj.weight"].T).view(T, c["kv_heads"], c["head_dim"])
            v = (h @ w[p + "self_attn.v_proj.weight"].T).view(T, c["kv_heads"], c["head_dim"])
            o = plain_llama.causal_attention(q, k, v, c["head_dim"] ** -0.5, softcap=cap, slopes=slopes)
            x = x + o.reshape(T, -1) @ w[p + "self_attn.o_proj.weight"].T
            h = plain_llama.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"])
            x = x + plain_llama.gated_mlp(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                                          w[p + "mlp.down_proj.weight"])
        return (plain_llama.rms_norm(x, w["model.norm.weight"], c["eps"]) @ w["lm_head.weight"].T).numpy()

    return hf, w, reqs, plain
