from .attention import Attention, paged_attention
from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITION_ENCODINGS, Delta, FeedForward, Mixer,
                   PagedKVSpec, Part, Registry, StateSpec)
from .block import Block, PostNormBlock, PreNormBlock, ResidualStream
from .embedding import Embedding, OutputHead
from .ffn import DenseFFN
from .norm import LayerNorm, NoNorm, Norm, RMSNorm
from .position import LearnedPositions, NoPositions, PositionEncoding

__all__ = ["Attention", "BLOCKS", "Block", "Delta", "DenseFFN", "Embedding", "FEED_FORWARDS", "FeedForward",
           "LayerNorm", "LearnedPositions", "MIXERS", "Mixer", "NORMS", "NoNorm", "NoPositions", "Norm",
           "OutputHead", "POSITION_ENCODINGS", "PagedKVSpec", "Part", "PositionEncoding", "PostNormBlock",
           "PreNormBlock", "RMSNorm", "Registry", "ResidualStream", "StateSpec", "paged_attention"]
