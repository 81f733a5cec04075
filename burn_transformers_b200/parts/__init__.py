from .attention import CausalSelfAttention
from .base import Block, FeedForward, Mixer, Norm, Part, PositionEncoding
from .block import PreNormBlock
from .embedding import TiedReadout, TokenEmbedding
from .feed_forward import DenseFeedForward
from .norm import LayerNorm
from .position import LearnedPositions, NoPositions

__all__ = ["CausalSelfAttention", "Block", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "PreNormBlock",
           "TiedReadout", "TokenEmbedding", "DenseFeedForward", "LayerNorm", "LearnedPositions", "NoPositions"]
