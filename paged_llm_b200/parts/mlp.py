"""Gated feed-forward: down(act(gate(x)) * up(x)), no bias, act = SiLU
(reference: pagedllm/model/llama.py:163-171).  Gate and up are stacked into one
matrix [2*intermediate, hidden] when the weights are taken."""

from __future__ import annotations

import torch

from .base import FeedForward, LazyLinear, TensorSpec, register_feed_forward


@register_feed_forward("gated_mlp")
class GatedMLP(FeedForward):
    accepts_lazy_input = True

    def __init__(self, weights: dict[str, str], hidden_size: int, intermediate_size: int, activation: str = "silu"):
        if activation != "silu":
            raise ValueError(f"activation {activation!r} is not implemented (silu only)")
        self.hidden_size, self.intermediate_size, self.activation = hidden_size, intermediate_size, activation
        self.names = weights
        self.w_gate_up = None
        self.w_down = None

    def tensor_specs(self):
        h, i = self.hidden_size, self.intermediate_size
        return {
            self.names["gate_proj"]: TensorSpec((i, h)),
            self.names["up_proj"]: TensorSpec((i, h)),
            self.names["down_proj"]: TensorSpec((h, i)),
        }

    def load(self, tensors):
        self.w_gate_up = torch.cat([tensors[self.names["gate_proj"]], tensors[self.names["up_proj"]]], dim=0).contiguous()
        self.w_down = tensors[self.names["down_proj"]].contiguous()

    def bytes_read_per_step(self):
        return sum(w.numel() * w.element_size() for w in (self.w_gate_up, self.w_down))

    def forward(self, h, ctx):
        ops = ctx.ops
        return LazyLinear(ops.gated_silu_linear(h, self.w_gate_up), self.w_down)
