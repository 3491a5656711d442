"""The parts a model is put together from (see ``base`` for the interfaces)."""
from .attention import GQAttention
from .base import (FeedForward, KVCacheNeed, Mixer, Norm, Part, PositionEncoding, Runtime, StateNeed, WeightSpec)
from .block import Block
from .embedding import Embedding, OutputHead
from .linear import Linear
from .norm import RMSNorm
from .rope import RotaryEmbedding
from .swiglu import SwiGLU

__all__ = ["GQAttention", "FeedForward", "KVCacheNeed", "Mixer", "Norm", "Part", "PositionEncoding", "Runtime",
           "StateNeed", "WeightSpec", "Block", "Embedding", "OutputHead", "Linear", "RMSNorm", "RotaryEmbedding", "SwiGLU"]
