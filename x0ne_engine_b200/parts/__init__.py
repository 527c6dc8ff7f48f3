"""The parts layers are made of, and their registries."""
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, PART_REGISTRIES, POSITIONS, Block, BuildEnv,
                   CacheNeed, Embedding, FeedForward, Head, Mixer, Norm, Part, PositionEncoding, Registry)
from .linear import Linear
from . import attention, block, embedding, mlp, norm, rope  # noqa: F401  (registers the built-in parts)
from .attention import GQAttention
from .block import PreNormBlock
from .embedding import LMHead, TokenEmbedding
from .mlp import SwiGLU
from .norm import RMSNorm
from .rope import NoPosition, Rope, inv_freq_f32

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "PART_REGISTRIES", "POSITIONS", "Block",
           "BuildEnv", "CacheNeed", "Embedding", "FeedForward", "Head", "Mixer", "Norm", "Part", "PositionEncoding",
           "Registry", "Linear", "GQAttention",
           "PreNormBlock", "LMHead", "TokenEmbedding", "SwiGLU", "RMSNorm", "NoPosition", "Rope", "inv_freq_f32"]
