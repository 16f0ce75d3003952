"""Parts that a model is put together from: embedding, mixer, feed-forward, norm, position encoding,
their arrangement in a block, and the LM head.  Importing the package registers the built-in kinds."""

from . import attention, block, embedding, feed_forward, norm, position  # noqa: F401  (registration)
from .base import (FeedForward, KVCacheSpec, LayerCache, LogitsHead, Mixer, Norm, Part, PositionEncoding,
                   StateSpec, TensorSource, TokenEmbedding, build_block, build_embedding, build_feed_forward,
                   build_lm_head, build_mixer, build_norm, build_position, register_arrangement,
                   register_embedding, register_feed_forward, register_lm_head, register_mixer,
                   register_norm, register_position)
from .spec import (EmbeddingSpec, GQAAttentionSpec, LayerCall, LayerSpec, LMHeadSpec, ModelSpec,
                   NoPositionSpec, RMSNormSpec, RopeSpec, SwiGLUSpec)
