"""Interfaces of the parts a model is put together from, and their registries.

A model is data: a `ModelSpec` lists layers, each layer names a block
arrangement, a mixer, a feed-forward and a norm by registry key with their
sizes and constants as parameters, and a schedule lists the order in which
layers run.  `build_model` (models/causal_lm.py) turns the data into objects by
looking the keys up here.  A part never learns which architecture it belongs
to: it gets its own sizes, the names of its tensors, and at run time a
`StepContext`.

Adding a part = subclass the interface, decorate with `register_*`, and name
the key in a spec.  Nothing else in the package has to change.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch


# --------------------------------------------------------------------------- specs (data)

@dataclass
class PartSpec:
    """One part as data: registry key, parameters, and tensor names.

    `weights` maps the part's own short names (e.g. "q_proj") to the tensor
    names of the checkpoint (e.g. "model.layers.3.self_attn.q_proj.weight").
    """

    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    weights: dict[str, str] = field(default_factory=dict)


@dataclass
class LayerSpec:
    """One layer: how mixer, feed-forward and norms are arranged (`block`)."""

    block: str
    mixer: PartSpec
    feed_forward: PartSpec
    norms: dict[str, PartSpec]


@dataclass
class ScheduleEntry:
    """One run of a layer.  `layer` indexes `ModelSpec.layers`, so a layer may be
    named twice (its weights are shared, each run has a cache of its own).
    `cache_from` names an earlier schedule entry whose cache this run reads
    instead of keeping one itself."""

    layer: int
    cache_from: int | None = None


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: list[LayerSpec]
    schedule: list[ScheduleEntry]
    final_norm: PartSpec
    head: PartSpec
    positions: dict[str, PartSpec] = field(default_factory=dict)   # position encodings by name
    ignored_tensors: tuple[str, ...] = ()                          # name suffixes a checkpoint may carry


@dataclass(frozen=True)
class TensorSpec:
    """What a part expects of one checkpoint tensor.

    role: "matrix" (a GEMM operand: kept in the compute dtype), "vector" (norm
    weights and the like: a tensor stored in 32-bit stays 32-bit, else compute
    dtype), "table_int" (integer tables: int32).
    init: how the random-weights mode draws it: "normal", "norm" (1 or 1+noise).
    optional: may be absent from the checkpoint (e.g. a tied head).
    """

    shape: tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    optional: bool = False
    alias_of: str | None = None      # optional tensor that, when absent, is this other tensor


# --------------------------------------------------------------------------- cache needs

@dataclass(frozen=True)
class PagedKV:
    """The mixer keeps a key and a value vector per token, in pages.
    `window`: only the last `window` tokens are ever read (None: all)."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class FixedState:
    """The mixer keeps a state of fixed size per request (float32 by default)."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


# --------------------------------------------------------------------------- lazy branch outputs

@dataclass
class LazyLinear:
    """A branch output `input @ weight^T` that has not been computed yet.

    A mixer or feed-forward whose last operation is a projection may return this
    instead of a tensor.  The norm that consumes the branch can then let one
    kernel do projection + residual sum + normalisation; anything else calls
    `materialize`.  A part that returns a plain tensor works everywhere too."""

    input: torch.Tensor
    weight: torch.Tensor

    def materialize(self, ops) -> torch.Tensor:
        return ops.linear(self.input, self.weight)

    def rows(self, ops, idx: torch.Tensor) -> "LazyLinear":
        """The same branch for the rows `idx` only."""
        return LazyLinear(ops.gather_rows(self.input, idx), self.weight)


def materialize(branch, ops):
    return branch.materialize(ops) if isinstance(branch, LazyLinear) else branch


# --------------------------------------------------------------------------- interfaces

class Part:
    """Common to all parts: which tensors it wants and how it takes them."""

    # True if `forward` hands its input straight to the kernel library's products, which
    # also take a normalisation that has not been carried out yet (ops.materialize turns
    # one into a tensor).  Parts that look at their input themselves leave this False.
    accepts_lazy_input = False

    # True if `forward` only launches work on the step's stream from the step's device
    # metadata, so that a decode step may be captured once and replayed.  A part that reads
    # `ctx.host`, waits for the device (e.g. to count rows) or allocates by data sets it
    # False; a model with one such part runs every step eagerly.
    capturable = True

    def tensor_specs(self) -> dict[str, TensorSpec]:
        """Checkpoint tensor name -> expectation."""
        return {}

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        """Take (already cast, on device) tensors by checkpoint name.  A part may
        fuse them into its own layout here; names on disk stay the checkpoint's."""

    def bytes_read_per_step(self) -> int:
        """Weight bytes one step has to read (for roofline arithmetic)."""
        return 0


class Norm(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """Normalise rows of `x` (residual stream dtype) -> compute dtype."""
        raise NotImplementedError

    def add_forward(self, x: torch.Tensor, branch, ctx) -> torch.Tensor:
        """x += branch (in place, in the residual dtype), then normalise.  With
        branch None this is `forward`.  `branch` is a tensor or a `LazyLinear`."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Owns what positions turn into (for rotary: the cos/sin table)."""

    def prepare(self, max_positions: int, device, ops) -> None:
        raise NotImplementedError


class Embedding(Part):
    """Turns the step's token ids into the residual stream."""

    def forward(self, ids: torch.Tensor, ctx) -> torch.Tensor:
        """ids: [T] int32 -> [T, hidden] float32 (the residual dtype).  A spec may give the
        part a `position` parameter naming a position encoding; it arrives as the object."""
        raise NotImplementedError


class Head(Part):
    """Turns normalised rows into logits."""

    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        """h: [rows, hidden] in the compute dtype -> [rows, vocab] float32."""
        raise NotImplementedError


class Mixer(Part):
    """Mixes information between the tokens of a request (attention here)."""

    def cache_requirement(self) -> PagedKV | FixedState | None:
        return None

    def forward(self, h: torch.Tensor, ctx, cache) -> torch.Tensor:
        """h: [T, hidden] in the compute dtype, token-major over all requests of
        the step.  `cache` is a `LayerCache` view (cache/storage.py) for this run
        of the layer, or None if the mixer keeps nothing.  Returns [T, hidden]
        (a tensor, or a `LazyLinear` if the last operation is a projection)."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, h: torch.Tensor, ctx) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """Arrangement of norms, mixer and feed-forward around the residual stream.

    The stream is a pair (x, pending): `x` in the residual dtype and a branch
    output not yet added, so that the sum can be fused with the next norm.
    """

    def __init__(self, mixer: Mixer, feed_forward: FeedForward, norms: dict[str, Norm]):
        self.mixer, self.feed_forward, self.norms = mixer, feed_forward, norms

    def forward(self, x, pending, ctx, cache):
        raise NotImplementedError

    def tensor_specs(self):
        out = {}
        for part in (self.mixer, self.feed_forward, *self.norms.values()):
            out.update(part.tensor_specs())
        return out

    def load(self, tensors):
        for part in (self.mixer, self.feed_forward, *self.norms.values()):
            part.load(tensors)

    def bytes_read_per_step(self):
        return sum(p.bytes_read_per_step() for p in (self.mixer, self.feed_forward, *self.norms.values()))

    @property
    def capturable(self):
        return all(p.capturable for p in (self.mixer, self.feed_forward, *self.norms.values()))


# --------------------------------------------------------------------------- registries

MIXERS: dict[str, Callable[..., Mixer]] = {}
FEED_FORWARDS: dict[str, Callable[..., FeedForward]] = {}
NORMS: dict[str, Callable[..., Norm]] = {}
POSITION_ENCODINGS: dict[str, Callable[..., PositionEncoding]] = {}
BLOCKS: dict[str, Callable[..., Block]] = {}
EMBEDDINGS: dict[str, Callable[..., Embedding]] = {}
HEADS: dict[str, Callable[..., Head]] = {}


def _register(table: dict, what: str):
    def outer(name: str):
        def inner(cls):
            if name in table and table[name] is not cls:
                raise ValueError(f"{what} {name!r} is already registered")
            table[name] = cls
            return cls
        return inner
    return outer


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position_encoding = _register(POSITION_ENCODINGS, "position encoding")
register_block = _register(BLOCKS, "block")
register_embedding = _register(EMBEDDINGS, "embedding")
register_head = _register(HEADS, "head")


def make_part(table: dict, what: str, spec: PartSpec, **extra):
    """Look a part up by its key and construct it from its spec."""
    try:
        cls = table[spec.kind]
    except KeyError:
        raise KeyError(f"unknown {what} {spec.kind!r}; registered: {sorted(table)}") from None
    return cls(weights=spec.weights, **spec.params, **extra)
