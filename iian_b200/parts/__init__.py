"""Parts a layer is put together from.  Importing the package registers the built-in kinds."""
from . import attention, block, chunked_attention, delta_rule, embedding, experts, latent_attention, matrix_memory, mlp, norm, position, shared_kv_attention, stream  # noqa: F401
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, STREAM_PARTS, KVNeed, RowNeed, StateNeed,  # noqa: F401
                   register_block, register_embedding, register_feed_forward, register_head, register_mixer,
                   register_norm, register_position, register_stream_part)
