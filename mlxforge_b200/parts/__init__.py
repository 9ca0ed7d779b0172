from .base import (BLOCKS, CONNECTIONS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, POSITIONS, Block, Connection,
                   DeltaPair, FeedForward,
                   FixedState, LayerSpec, Mixer, ModelSpec, Norm, PagedKV, Part, PartSpec, PositionEncoding,
                   ScaledPair, ScheduleItem, TensorSpec, build_part, register_block, register_connection, register_embedding,
                   register_feed_forward, register_head, register_mixer, register_norm, register_position)
from . import (attention, block, connections, delta_rule, embedding, latent_attention, mlp, moe, norms,  # noqa: F401
               retention, rope, side_by_side, talking_attention)                                                  # (register the built-in parts)
