"""Parts that a model is put together from: embedding, mixer, feed-forward, norm, position encoding,
their arrangement in a block, and the LM head.  Importing the package registers the built-in kinds."""

from . import (attention, biased_attention, block, embedding, feed_forward, gated_delta, latent_attention,  # noqa: F401  (registration)
               lightning, linear_recurrence, norm, parallel, position, routed_ff)
from .base import (FeedForward, KVCacheSpec, LayerCache, LogitsHead, Mixer, Norm, Part, PositionEncoding,
                   StateSpec, TensorSource, TokenEmbedding, build_block, build_embedding, build_feed_forward,
                   build_lm_head, build_mixer, build_norm, build_position, register_arrangement,
                   register_embedding, register_feed_forward, register_lm_head, register_mixer,
                   register_norm, register_position)
from .spec import (BiasedAttentionSpec, DenseFFSpec, DistanceBiasSpec, EmbeddingSpec, ForgetGateRecurrenceSpec, GatedDeltaSpec, GQAAttentionSpec, LatentAttentionSpec, LayerCall, LayerSpec,
                   LightningAttentionSpec, LMHeadSpec, ModelSpec, NoPositionSpec, ParallelMixerSpec, RetentionSpec, RMSNormSpec, RopeSpec,
                   RoutedFFSpec, SwiGLUSpec, YarnRopeSpec)
