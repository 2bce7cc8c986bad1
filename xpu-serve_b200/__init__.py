"""A B200-native model library for LFM3: from a request's tokens to its next token.

Import as `xpu_serve_b200`. Importing the package needs no GPU; the CUDA extension is
compiled and loaded when a model is first put on a device.
"""
__version__ = "0.1.0"

from . import registry                                   # noqa: E402
from .config import ConfigError, Lfm3Config              # noqa: E402
from . import parts                                      # noqa: E402,F401  (registers the parts)

registry.register_architecture("lfm3", Lfm3Config, aliases=("lfm3_vl", "Lfm3ForCausalLM"))


def load_model(folder, dtype="bfloat16", device="cuda:0"):
    """The model that the folder's config.json names, ready to step on `device`."""
    from .engine.model import load_model as _load
    return _load(folder, dtype=dtype, device=device)

from .sampling import GenerateRequest, GenerateResult, GenerateStats, SamplingParams   # noqa: E402


def __getattr__(name):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    raise AttributeError(name)
