"""Parts a layer is put together from.  Importing the package registers the built-in kinds."""
from . import (attention, block, chunked_attention, delta_rule, embedding, experts, latent_attention, linear_attention,  # noqa: F401
               matrix_memory, mlp, norm, position, shared_kv_attention, side_by_side, stream, window_attention)
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, STREAM_PARTS, KVNeed, RowNeed, StateNeed,  # noqa: F401
                   register_block, register_embedding, register_feed_forward, register_head, register_mixer,
                   register_norm, register_position, register_stream_part)
