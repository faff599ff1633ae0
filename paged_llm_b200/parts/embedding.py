"""Token embedding and the output head.

x[t] = E[ids[t]] with no scaling (reference: pagedllm/model/llama.py:191, :197);
logits = h W^T in float32, where W is E itself if the head is tied
(llama.py:208-216).  A tied checkpoint may still carry the head's tensor; it is
then ignored, as tying means the embedding is used.
"""

from __future__ import annotations

from .base import Embedding, Head, TensorSpec, register_embedding, register_head


@register_embedding("embedding")
class TokenEmbedding(Embedding):
    def __init__(self, weights: dict[str, str], vocab_size: int, hidden_size: int):
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.name = weights["weight"]
        self.weight = None

    def tensor_specs(self):
        return {self.name: TensorSpec((self.vocab_size, self.hidden_size))}

    def load(self, tensors):
        self.weight = tensors[self.name].contiguous()

    def forward(self, ids, ctx):
        return ctx.ops.embedding(self.weight, ids)


@register_head("lm_head")
class LMHead(Head):
    accepts_lazy_input = True

    def __init__(self, weights: dict[str, str], vocab_size: int, hidden_size: int, tied_to: str | None = None):
        self.vocab_size, self.hidden_size = vocab_size, hidden_size
        self.name = weights["weight"]
        self.tied_to = tied_to
        self.weight = None

    def tensor_specs(self):
        return {self.name: TensorSpec((self.vocab_size, self.hidden_size), optional=self.tied_to is not None,
                                      alias_of=self.tied_to)}

    def load(self, tensors):
        self.weight = (tensors[self.tied_to] if self.tied_to is not None else tensors[self.name]).contiguous()

    def bytes_read_per_step(self):
        return self.weight.numel() * self.weight.element_size()

    def forward(self, h, ctx):
        return ctx.ops.linear(h, self.weight, out_float32=True)
