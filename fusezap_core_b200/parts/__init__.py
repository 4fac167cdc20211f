from .base import (MIXERS, FEED_FORWARDS, NORMS, POSITIONS, BLOCKS, LOGIT_TRANSFORMS, EMBED_EXTRAS, register_mixer, register_feed_forward,
                   register_norm, register_position, register_block, register_logit_transform, register_embed_extra,
                   build, LayerCache, Part, Mixer, FeedForward, Norm, PositionEncoding, Block, LogitTransform, EmbedExtra)
from . import rope, norm, attention, feed_forward, block   # registers the dense decoder's parts
from . import short_conv, parallel_block, latent_attention, table_moe, logit   # gated parallel block, latent attention, table-routed experts
from . import retention, sink_attention, gated_delta, parallel_mixers, routed_moe   # recurrent mixers, windowed attention with a sink, routed experts
from . import hashed_pair, depth_average, general_delta   # hashed pair embedding, depth-averaged layers, generalized delta rule
from . import rglru   # real-gated linear recurrent unit

__all__ = ["MIXERS", "FEED_FORWARDS", "NORMS", "POSITIONS", "BLOCKS", "LOGIT_TRANSFORMS", "EMBED_EXTRAS", "register_mixer",
           "register_feed_forward", "register_norm", "register_position", "register_block", "register_logit_transform", "register_embed_extra",
           "build", "LayerCache", "Part", "Mixer", "FeedForward", "Norm", "PositionEncoding", "Block", "LogitTransform", "EmbedExtra"]
