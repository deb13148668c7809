from .base import (KVRequest, ParamSpec, StateRequest, block_class, feed_forward_class,
                   mixer_class, norm_class, position_class, register_block,
                   register_feed_forward, register_mixer, register_norm, register_position,
                   register_stream_position, stream_position_class)
from .norm import Identity, LayerNorm, RMSNorm
from .rope import RotaryEmbedding
from .attention import AttentionMixer
from .latent import LatentAttentionMixer
from .delta import ChannelDeltaMixer
from .position import LearnedPosition
from .feedforward import DenseFeedForward, GatedFeedForward
from .moe import RoutedFeedForward
from .block import Block
from .linear import GatedLinear, Linear

__all__ = ["KVRequest", "ParamSpec", "StateRequest", "feed_forward_class", "mixer_class",
           "norm_class", "position_class", "block_class", "stream_position_class",
           "register_block", "register_feed_forward", "register_mixer", "register_norm",
           "register_position", "register_stream_position", "RMSNorm", "LayerNorm",
           "RoutedFeedForward", "RotaryEmbedding", "Identity", "LatentAttentionMixer",
           "DenseFeedForward", "ChannelDeltaMixer", "LearnedPosition",
           "AttentionMixer", "GatedFeedForward", "Block", "GatedLinear", "Linear"]
