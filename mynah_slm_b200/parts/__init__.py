"""Parts a layer is put together from. Importing the package registers the
built-in ones."""
from .base import (Block, CacheView, Embedding, FeedForward, Head, KVRequest, Mixer, Norm, Part, PositionEncoding,
                   Residual, StateRequest, TensorSpec, build_part, known_parts, register_block,
                   register_embedding, register_ffn, register_head, register_mixer, register_norm,
                   register_position)
from . import attention, block, embedding, feedforward, norms, position  # noqa: F401  (registration)
from .embedding import LinearHead, TokenEmbedding
