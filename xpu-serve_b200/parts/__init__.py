"""The parts a layer is put together from. Importing this package registers them."""
from .base import FeedForward, KVNeed, Mixer, Part, StateNeed, TensorSpec
from .rope import RotaryTable
from .attention import AttentionMixer
from .short_conv import ShortConvMixer
from .swiglu import SwiGLU
from .block import Block, ResidualStream

__all__ = ["FeedForward", "KVNeed", "Mixer", "Part", "StateNeed", "TensorSpec", "RotaryTable",
           "AttentionMixer", "ShortConvMixer", "SwiGLU", "Block", "ResidualStream"]
