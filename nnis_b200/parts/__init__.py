from . import attention, block, embedding, mlp, norm, position  # noqa: F401  (registration)
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, Part, Registry
from .embedding import LinearHead, TokenEmbedding
from .linear import ADD_F32, STORE, STORE_F32, linear

__all__ = ["BLOCKS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "Part", "Registry",
           "LinearHead", "TokenEmbedding", "ADD_F32", "STORE", "STORE_F32", "linear"]
