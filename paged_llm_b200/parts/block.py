"""Pre-norm arrangement: x += mixer(norm_in(x)); x += ffn(norm_post(x))
(reference: pagedllm/model/llama.py:174-185).  Each residual sum is handed to
the following norm as a pending branch so that one kernel does both."""

from __future__ import annotations

from .base import Block, register_block


@register_block("pre_norm")
class PreNormBlock(Block):
    NORM_NAMES = ("input", "post_mixer")

    def forward(self, x, pending, ctx, cache):
        h = self.norms["input"].add_forward(x, pending, ctx)
        if not self.mixer.accepts_lazy_input:
            h = ctx.ops.materialize(h)
        a = self.mixer.forward(h, ctx, cache)
        h = self.norms["post_mixer"].add_forward(x, a, ctx)
        if not self.feed_forward.accepts_lazy_input:
            h = ctx.ops.materialize(h)
        f = self.feed_forward.forward(h, ctx)
        return x, f
