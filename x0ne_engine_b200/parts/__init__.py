"""The parts layers are made of, and their registries."""
from .base import (BLOCKS, EMBEDDINGS, FEED_FORWARDS, HEADS, MIXERS, NORMS, PART_REGISTRIES, POSITIONS, Block, BuildEnv,
                   CacheNeed, Embedding, FeedForward, Head, Mixer, Norm, Part, PositionEncoding, Registry)
from .linear import Linear
from . import attention, block, embedding, latent_attention, masked_attention, mlp, norm, rope  # noqa: F401  (registers the built-in parts)
from .attention import GQAttention
from .block import ParallelBlock, PreNormBlock
from .latent_attention import LatentAttention
from .masked_attention import MaskedAttention
from .embedding import LMHead, TokenEmbedding
from .mlp import ClippedGLU, SwiGLU
from .norm import RMSNorm
from .rope import NoPosition, Rope, YarnRope, inv_freq_f32, yarn_frequencies

__all__ = ["BLOCKS", "EMBEDDINGS", "FEED_FORWARDS", "HEADS", "MIXERS", "NORMS", "PART_REGISTRIES", "POSITIONS", "Block",
           "BuildEnv", "CacheNeed", "Embedding", "FeedForward", "Head", "Mixer", "Norm", "Part", "PositionEncoding",
           "Registry", "Linear", "GQAttention",
           "PreNormBlock", "ParallelBlock", "MaskedAttention", "LatentAttention", "ClippedGLU", "YarnRope", "yarn_frequencies", "LMHead", "TokenEmbedding", "SwiGLU", "RMSNorm", "NoPosition", "Rope", "inv_freq_f32"]
