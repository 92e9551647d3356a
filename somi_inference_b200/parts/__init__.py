"""Parts of a decoder layer, their registries, and the generic decoder built from them."""

from . import block, embedding, feedforward, mixer, norm, position  # noqa: F401  (register kinds)
from .base import BuildContext, CacheNeeds, PagedKVNeeds, StateNeeds, TensorDecl
from .model import Decoder, declared_tensors
from .registry import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS,
                       POSITION_ENCODINGS)

__all__ = ["BuildContext", "CacheNeeds", "PagedKVNeeds", "StateNeeds", "TensorDecl", "Decoder",
           "declared_tensors", "ARRANGEMENTS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS",
           "NORMS", "POSITION_ENCODINGS"]
