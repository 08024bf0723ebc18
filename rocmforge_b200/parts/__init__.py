from .base import (Part, Norm, PositionEncoding, Mixer, FeedForward, Block, Registry,
                   NORMS, POSITIONS, MIXERS, FEED_FORWARDS, BLOCKS)
from .linear import Linear
from .norm import RMSNorm
from .rope import NeoxRope
from .attention import GQAAttention
from .mlp import GatedMLP
from .block import PreNormBlock
from .embedding import TokenEmbedding, OutputHead
