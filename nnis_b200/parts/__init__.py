from . import attention, block, embedding, mlp, norm, position  # noqa: F401  (registration)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Part,
                   PositionEncoding, Registry)
from .block import Block
from .embedding import LinearHead, TokenEmbedding
from .linear import ADD_F32, STORE, STORE_F32, linear

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "POSITIONS", "Part",
           "PositionEncoding", "Registry", "Block", "LinearHead", "TokenEmbedding", "ADD_F32", "STORE",
           "STORE_F32", "linear"]
