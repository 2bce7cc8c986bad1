"""Typed configurations and the architecture-neutral model description."""
from .json_util import ConfigError, read_json
from .lfm3 import Lfm3Config, Lfm3Rope
from .spec import (AttentionSpec, LayerCall, LayerSpec, ModelSpec, NormSpec, RopeSpec,
                   ShortConvSpec, SwiGLUSpec)

__all__ = ["ConfigError", "read_json", "Lfm3Config", "Lfm3Rope", "AttentionSpec", "LayerCall",
           "LayerSpec", "ModelSpec", "NormSpec", "RopeSpec", "ShortConvSpec", "SwiGLUSpec"]
