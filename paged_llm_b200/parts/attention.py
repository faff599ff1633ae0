"""Grouped-query attention over the paged cache.

q, k, v = h Wq^T, h Wk^T, h Wv^T (no bias), rotary on q and k, k and v written to
their slots of the cache, attention through the block table with query head h
reading kv head h // (heads // kv_heads), then the output projection
(reference: pagedllm/model/llama.py:131-160; the attention itself:
pagedllm/attention/reference.py:23-55).  The three projections are stacked into
one matrix when the weights are taken, so a step runs one product for them.

`scale` and `window` are parameters: the reference fixes scale = head_dim^-0.5
(llama.py:138) and has no window; a window w keeps, for the query at position p,
the keys at positions p-w+1 .. p.  Two score modifiers, off unless a spec asks
for them (the reference has neither): `score_cap` c turns a scaled score s into
c * tanh(s / c), and `position_slopes` (one number per query head) adds
slope * (key position - query position) to it, a bias by distance that needs no
rotation of q and k.
"""

from __future__ import annotations

import torch

from .base import LazyLinear, Mixer, PagedKV, TensorSpec, register_mixer


@register_mixer("paged_attention")
class PagedAttention(Mixer):
    accepts_lazy_input = True

    def __init__(self, weights: dict[str, str], hidden_size: int, num_heads: int, num_kv_heads: int,
                 head_dim: int, scale: float | None = None, window: int | None = None, position=None,
                 score_cap: float | None = None, position_slopes=None):
        if num_heads % num_kv_heads:
            raise ValueError(f"num_heads={num_heads} is not a multiple of num_kv_heads={num_kv_heads}")
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.window = window
        self.position = position
        if score_cap is not None and not score_cap > 0:
            raise ValueError(f"score_cap={score_cap} must be positive")
        if position_slopes is not None and len(position_slopes) != num_heads:
            raise ValueError(f"position_slopes has {len(position_slopes)} entries for {num_heads} heads")
        self.score_cap = score_cap
        self.position_slopes = [float(x) for x in position_slopes] if position_slopes is not None else None
        self._slopes = None              # the same on the device, made at the first step
        self.names = weights
        self.w_qkv = None
        self.w_o = None

    def cache_requirement(self):
        return PagedKV(self.num_kv_heads, self.head_dim, self.window)

    def attention_plan_key(self):
        """(query heads per kv head, kv heads, window, head size): what the step's work lists depend on."""
        return (self.num_heads // self.num_kv_heads, self.num_kv_heads, self.window, self.head_dim)

    def tensor_specs(self):
        h, d = self.hidden_size, self.head_dim
        return {
            self.names["q_proj"]: TensorSpec((self.num_heads * d, h)),
            self.names["k_proj"]: TensorSpec((self.num_kv_heads * d, h)),
            self.names["v_proj"]: TensorSpec((self.num_kv_heads * d, h)),
            self.names["o_proj"]: TensorSpec((h, self.num_heads * d)),
        }

    def load(self, tensors):
        self.w_qkv = torch.cat([tensors[self.names[k]] for k in ("q_proj", "k_proj", "v_proj")], dim=0).contiguous()
        self.w_o = tensors[self.names["o_proj"]].contiguous()

    def bytes_read_per_step(self):
        return sum(w.numel() * w.element_size() for w in (self.w_qkv, self.w_o))

    def forward(self, h, ctx, cache):
        ops = ctx.ops
        block_table = ctx.block_tables[cache.group]
        if self.position_slopes is not None and self._slopes is None:
            self._slopes = torch.tensor(self.position_slopes, dtype=torch.float32, device=cache.kv.device)
        o = ops.qkv_attention(h, self.w_qkv, self.num_heads, self.num_kv_heads, self.head_dim, self.position, ctx,
                              cache.kv, block_table, self.scale, self.window, write=cache.owner,
                              softcap=self.score_cap, slopes=self._slopes)
        return LazyLinear(o, self.w_o)
