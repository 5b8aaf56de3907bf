"""Parts a model is put together from: norms, position encodings, mixers, feed-forwards, blocks."""
from .base import (KVNeed, StateNeed, LayerCache, StepContext, Part, Norm, PositionEncoding, Mixer, FeedForward, Block,
                   register_mixer, register_feed_forward, register_norm, register_position_encoding,
                   make_mixer, make_feed_forward, make_norm, make_position_encoding,
                   MIXERS, FEED_FORWARDS, NORMS, POSITION_ENCODINGS)
from .norm import RMSNorm, DynamicTanh
from .rotary import RotaryEncoding, ScaledRotaryEncoding, BandRotaryEncoding
from .attention import AttentionMixer
from .latent_attention import LatentAttentionMixer
from .bias_attention import BiasedWindowAttentionMixer
from .gated_attention import RotatedValueAttentionMixer, DifferentialAttentionMixer
from .delta import ChannelDeltaMixer
from .ssm import Mamba2Mixer
from .retention import RetentionMixer
from .parallel import ParallelMixer
from .token_side import TokenSideInput
from .dense_ffn import SwiGLUFeedForward, ReluSquaredFeedForward, GluFeedForward
from .moe_ffn import MoEFeedForward
from .block import PreNormBlock, PostNormBlock, SandwichBlock, DepthMixBlock
