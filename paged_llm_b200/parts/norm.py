"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, all in 32-bit, eps inside the
root, the weight multiplied before the down-cast (reference:
pagedllm/model/llama.py:74-83)."""

from __future__ import annotations

from .base import LazyLinear, Norm, TensorSpec, register_norm


@register_norm("rms_norm")
class RMSNorm(Norm):
    def __init__(self, weights: dict[str, str], dim: int, eps: float):
        self.dim, self.eps = dim, float(eps)
        self.name = weights["weight"]
        self.weight = None

    def tensor_specs(self):
        return {self.name: TensorSpec((self.dim,), role="vector", init="norm")}

    def load(self, tensors):
        self.weight = tensors[self.name].contiguous()

    def bytes_read_per_step(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, x, ctx):
        return ctx.ops.rms_norm(x, self.weight, self.eps)

    def add_forward(self, x, branch, ctx):
        if branch is None:
            return ctx.ops.rms_norm(x, self.weight, self.eps)
        if isinstance(branch, LazyLinear):
            return ctx.ops.linear_add_rms_norm(branch.input, branch.weight, x, self.weight, self.eps)
        return ctx.ops.add_rms_norm(x, branch, self.weight, self.eps)
