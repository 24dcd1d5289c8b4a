"""The parts a model is put together from; importing the package registers the
built-in kinds."""
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITION_ENCODINGS, Block, Embedding,
                   FeedForward, Head, Mixer, Norm, PagedKVNeed, Part, PartSpec, PositionEncoding, StateNeed,
                   WeightDecl, register_block, register_embedding, register_feed_forward, register_head,
                   register_mixer, register_norm, register_position_encoding)
from . import attention, block, embedding, ffn, norm, rope, shortconv  # noqa: F401  (registration)
