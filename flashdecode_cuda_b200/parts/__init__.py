"""The parts a model is put together from.  Importing this package registers
the parts of the architectures this library ships."""

from . import (attention, block, conv_attention, embedding, head, lanes, mlp, moe, norm, normed_attention,  # noqa: F401
               parallel, recurrent, rope, side, stream)  # noqa: F401  (registration)
from .base import (Block, Embedding, FeedForward, Head, KVRequest, LayerCache, Mixer, Norm, Part, Position,
                   Runtime)

__all__ = ["Part", "Embedding", "Position", "Norm", "Mixer", "FeedForward", "Block", "Head", "Runtime",
           "KVRequest", "LayerCache"]
