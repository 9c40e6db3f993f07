"""Parts a layer is put together from; importing this package registers the built-in kinds."""
from . import (attention, block, delta_rule, diff_attention, embedding, gla, latent_attention, mlp, moe, norm, rglru, rope,
               side_by_side, ssm)  # noqa: F401
from .base import (BLOCKS, CONNECTIONS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS, CacheSpec, TensorDecl, register_block,
                   register_connection, register_feed_forward, register_mixer, register_norm, register_position)

__all__ = ["BLOCKS", "CONNECTIONS", "FEED_FORWARDS", "MIXERS", "NORMS", "POSITIONS", "CacheSpec", "TensorDecl", "register_block", "register_connection",
           "register_feed_forward", "register_mixer", "register_norm", "register_position"]
