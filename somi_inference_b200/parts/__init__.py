"""Parts of a decoder layer, their registries, and the generic decoder built from them."""

from . import (block, conv_attention, embedding, extras, feedforward, latent, mamba2, mixer, moe,  # noqa: F401
               norm, position)                                    # (register kinds)
from .base import (BuildContext, CacheNeeds, GatedDelta, NormedDelta, PagedKVNeeds, StateNeeds,
                   TensorDecl)
from .model import Decoder, declared_tensors
from .registry import (ARRANGEMENTS, EMBEDDINGS, FEED_FORWARDS, HEADS, LAYER_EXTRAS, MIXERS, NORMS,
                       POSITION_ENCODINGS)

__all__ = ["BuildContext", "CacheNeeds", "GatedDelta", "NormedDelta", "PagedKVNeeds", "StateNeeds", "TensorDecl", "Decoder",
           "declared_tensors", "ARRANGEMENTS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "LAYER_EXTRAS", "MIXERS",
           "NORMS", "POSITION_ENCODINGS"]
