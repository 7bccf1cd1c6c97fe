from .base import (Block, CacheSpec, FeedForward, FixedStateSpec, Mixer, Norm, PagedKVSpec, Part,
                   PositionEncoding, Rotation, WeightSlot)
from .linear import Linear
from .norm import RMSNorm
from .rotary import NoPositionEncoding, RotaryHalf, RotaryInterleaved, SinusoidalPositions
from .attention import GroupedQueryAttention
from .mlp import GatedMLP
from .attention_gated import GatedWindowAttention
from .attention_latent import LatentAttention
from .delta import ChannelDeltaMixer
from .moe import RoutedExperts
from .side_input import TokenSideInput, TokenTable
from .block import ParallelBlock, PreNormBlock
from .embedding import LMHead, TokenEmbedding

__all__ = ["Block", "CacheSpec", "FeedForward", "FixedStateSpec", "Mixer", "Norm", "PagedKVSpec", "Part",
           "PositionEncoding", "Rotation", "WeightSlot", "Linear", "RMSNorm", "NoPositionEncoding", "RotaryHalf", "RotaryInterleaved",
           "GroupedQueryAttention", "GatedMLP", "PreNormBlock", "LMHead", "TokenEmbedding", "SinusoidalPositions",
           "GatedWindowAttention", "LatentAttention", "ChannelDeltaMixer", "RoutedExperts", "TokenSideInput", "TokenTable", "ParallelBlock"]
