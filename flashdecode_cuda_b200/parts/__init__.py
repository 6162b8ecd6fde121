"""The parts a model is put together from.  Importing this package registers
the parts of the Qwen2 dense decoder."""

from . import attention, block, embedding, head, mlp, norm, rope  # noqa: F401  (registration)
from .base import (Block, Embedding, FeedForward, Head, KVRequest, LayerCache, Mixer, Norm, Part, Position,
                   Runtime)

__all__ = ["Part", "Embedding", "Position", "Norm", "Mixer", "FeedForward", "Block", "Head", "Runtime",
           "KVRequest", "LayerCache"]
