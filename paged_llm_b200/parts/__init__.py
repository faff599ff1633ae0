"""Parts a model is assembled from.  Importing the package registers the
built-in ones."""

from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, Embedding, FeedForward, FixedState,
                   Head, LayerSpec, LazyLinear, materialize, Mixer, ModelSpec, Norm, PagedKV, Part, PartSpec, PositionEncoding, ScheduleEntry,
                   TensorSpec, make_part, register_block, register_embedding, register_feed_forward, register_head, register_mixer, register_norm,
                   register_position_encoding)
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registration)

__all__ = [
    "BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITION_ENCODINGS", "Block", "Embedding", "FeedForward", "FixedState",
    "Head", "LayerSpec", "LazyLinear", "materialize", "Mixer", "ModelSpec", "Norm", "PagedKV", "Part", "PartSpec", "PositionEncoding", "ScheduleEntry",
    "TensorSpec", "make_part", "register_block", "register_embedding", "register_feed_forward", "register_head", "register_mixer", "register_norm",
    "register_position_encoding",
]
