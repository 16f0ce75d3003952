"""Parts that layers are put together from: mixer, feed-forward, norm, position encoding, and
their arrangement in a block.  Importing the package registers the built-in kinds."""

from . import attention, block, feed_forward, norm, position  # noqa: F401  (registration)
from .base import (FeedForward, KVCacheSpec, LayerCache, Mixer, Norm, Part, PositionEncoding,
                   StateSpec, TensorSource, build_block, build_feed_forward, build_mixer,
                   build_norm, build_position, register_arrangement, register_feed_forward,
                   register_mixer, register_norm, register_position)
from .spec import (GQAAttentionSpec, LayerCall, LayerSpec, ModelSpec, NoPositionSpec, RMSNormSpec,
                   RopeSpec, SwiGLUSpec)
