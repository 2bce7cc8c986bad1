"""The parts a layer is put together from. Importing this package registers them."""
from .base import FeedForward, KVNeed, Mixer, Norm, Part, StateNeed, TensorSpec
from .norm import RMSNorm
from .rope import RotaryTable
from .attention import AttentionMixer
from .short_conv import ShortConvMixer
from .swiglu import SwiGLU
from .block import Block, ResidualStream

__all__ = ["FeedForward", "KVNeed", "Mixer", "Norm", "RMSNorm", "Part", "StateNeed", "TensorSpec", "RotaryTable",
           "AttentionMixer", "ShortConvMixer", "SwiGLU", "Block", "ResidualStream"]
