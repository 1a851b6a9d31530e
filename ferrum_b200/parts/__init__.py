from .attention import PagedAttention
from .base import (CacheNeed, FeedForward, Mixer, Norm, PagedKVNeed, ParamSpec, Part, PositionEncoding,
                   StateNeed)
from .block import (ParallelBlock, ParallelGatedBlock, PostNormBlock, PreNormBlock, StreamBlock, StreamSumNorm, TokenSideInput,
                    TokenSideTable)
from .embedding import LearnedPositions, OutputHead, TokenEmbedding
from .latent_attention import LatentAttention
from .ffn import RoutedFeedForward, SwiGLU
from .delta_rule import ChannelDeltaMixer
from .mamba2 import Mamba2Mixer
from .matrix_memory import MatrixMemoryMixer
from .parallel_mixer import ParallelMixer
from .shaped_attention import ShapedAttention
from .norm import RMSNorm
from .rope import RotaryEmbedding

__all__ = ["PagedAttention", "CacheNeed", "FeedForward", "Mixer", "Norm", "PagedKVNeed", "ParamSpec", "Part",
           "PositionEncoding", "StateNeed", "PreNormBlock", "ParallelGatedBlock", "LatentAttention", "LearnedPositions", "OutputHead", "TokenEmbedding", "SwiGLU", "RMSNorm",
           "RotaryEmbedding", "ParallelBlock", "TokenSideInput", "TokenSideTable", "Mamba2Mixer", "ShapedAttention", "StreamBlock", "StreamSumNorm",
           "RoutedFeedForward", "PostNormBlock", "ChannelDeltaMixer", "MatrixMemoryMixer", "ParallelMixer"]
