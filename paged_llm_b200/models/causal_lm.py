"""A causal language model assembled from a `ModelSpec`.

Embedding -> the scheduled runs of layers -> final norm on the wanted rows ->
head (reference: pagedllm/model/llama.py:188-216).  Unlike the reference, which
normalises all rows and then selects (llama.py:200, :216), rows are selected
first; the result is the same.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..parts.base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, FixedState,
                          LazyLinear, ModelSpec, PagedKV, PartSpec, TensorSpec, make_part)


@dataclass(frozen=True)
class CacheSlot:
    """What one scheduled run of a layer needs from the cache manager."""

    entry: int                                   # index into the schedule
    requirement: PagedKV | FixedState | None
    shares: int | None                           # schedule entry whose cache is read instead


def _resolve_positions(spec: PartSpec, positions: dict) -> dict:
    extra = {}
    params = dict(spec.params)
    if "position" in params:
        name = params.pop("position")
        extra["position"] = positions[name] if name is not None else None
    return PartSpec(spec.kind, params, spec.weights), extra


class CausalLM:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.positions = {name: make_part(POSITION_ENCODINGS, "position encoding", ps)
                          for name, ps in spec.positions.items()}
        emb_spec, extra = _resolve_positions(spec.embedding, self.positions)
        self.embedding = make_part(EMBEDDINGS, "embedding", emb_spec, **extra)
        self.blocks = []
        for layer in spec.layers:
            mixer_spec, extra = _resolve_positions(layer.mixer, self.positions)
            mixer = make_part(MIXERS, "mixer", mixer_spec, **extra)
            ffn = make_part(FEED_FORWARDS, "feed-forward", layer.feed_forward)
            norms = {k: make_part(NORMS, "norm", ns) for k, ns in layer.norms.items()}
            try:
                block_cls = BLOCKS[layer.block]
            except KeyError:
                raise KeyError(f"unknown block {layer.block!r}; registered: {sorted(BLOCKS)}") from None
            self.blocks.append(block_cls(mixer, ffn, norms))
        self.final_norm = make_part(NORMS, "norm", spec.final_norm)
        self.head = make_part(HEADS, "head", spec.head)
        self.schedule = list(spec.schedule)
        for i, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.blocks):
                raise ValueError(f"schedule entry {i} names layer {entry.layer}, there are {len(self.blocks)}")
            if entry.cache_from is not None:
                if not 0 <= entry.cache_from < i or self.schedule[entry.cache_from].cache_from is not None:
                    raise ValueError(f"schedule entry {i}: cache_from must name an earlier entry that owns a cache")
                mine = self.blocks[entry.layer].mixer.cache_requirement()
                theirs = self.blocks[self.schedule[entry.cache_from].layer].mixer.cache_requirement()
                if mine != theirs:
                    raise ValueError(f"schedule entry {i} cannot read the cache of entry {entry.cache_from}: "
                                     f"{mine} != {theirs}")

    # ---- weights ---------------------------------------------------------------
    def _parts(self):
        return [self.embedding, *self.blocks, self.final_norm, self.head, *self.positions.values()]

    def tensor_specs(self) -> dict[str, TensorSpec]:
        out: dict[str, TensorSpec] = {}
        for part in self._parts():
            for name, ts in part.tensor_specs().items():
                if name in out and out[name] != ts:
                    raise ValueError(f"tensor {name} is claimed twice with different expectations")
                out[name] = ts
        return out

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        for part in self._parts():
            part.load(tensors)

    def prepare(self, max_positions: int, device, ops) -> None:
        for pos in self.positions.values():
            pos.prepare(max_positions, device, ops)

    @property
    def capturable(self) -> bool:
        """True if every part allows a step to be captured and replayed."""
        return all(part.capturable for part in self._parts())

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights a decode step reads: every scheduled run reads its
        layer's matrices once, plus the head (the embedding is a gather)."""
        total = sum(self.blocks[e.layer].bytes_read_per_step() for e in self.schedule)
        return total + self.final_norm.bytes_read_per_step() + self.head.bytes_read_per_step()

    # ---- cache needs -----------------------------------------------------------
    def cache_slots(self) -> list[CacheSlot]:
        return [CacheSlot(i, self.blocks[e.layer].mixer.cache_requirement(), e.cache_from)
                for i, e in enumerate(self.schedule)]

    @property
    def has_fixed_state(self) -> bool:
        """True if a scheduled run keeps per-request state of fixed size (the engine then holds state slots)."""
        return any(isinstance(slot.requirement, FixedState) for slot in self.cache_slots())

    # ---- forward ---------------------------------------------------------------
    def forward(self, ctx) -> torch.Tensor | None:
        """Runs the tokens of `ctx` and returns float32 logits [wanted, vocab] at
        `ctx.logits_indices` (None if nothing is wanted)."""
        x = self.embedding.forward(ctx.input_ids, ctx)
        pending = None
        for i, entry in enumerate(self.schedule):
            x, pending = self.blocks[entry.layer].forward(x, pending, ctx, ctx.layer_caches[i])
        if ctx.num_logits == 0:
            return None
        ops = ctx.ops
        if getattr(ctx, "logits_all", False):
            # every row is wanted, in order: x may be finished in place, nothing to gather
            h = self.final_norm.add_forward(x, pending, ctx)
            if not self.head.accepts_lazy_input:
                h = ops.materialize(h)
            return self.head.forward(h, ctx)
        rows = ops.gather_rows(x, ctx.logits_indices)
        if pending is None:
            rows_pending = None
        elif isinstance(pending, LazyLinear):
            rows_pending = pending.rows(ops, ctx.logits_indices)     # the last projection runs on the wanted rows only
        else:
            rows_pending = ops.gather_rows(pending, ctx.logits_indices)
        h = self.final_norm.add_forward(rows, rows_pending, ctx)
        if not self.head.accepts_lazy_input:
            h = ops.materialize(h)
        return self.head.forward(h, ctx)


def build_model(spec: ModelSpec) -> CausalLM:
    return CausalLM(spec)
