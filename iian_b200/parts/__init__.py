"""Parts a layer is put together from.  Importing the package registers the built-in kinds."""
from . import attention, block, embedding, mlp, norm, position  # noqa: F401
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, KVNeed, StateNeed,  # noqa: F401
                   register_block, register_embedding, register_feed_forward, register_head, register_mixer,
                   register_norm, register_position)
