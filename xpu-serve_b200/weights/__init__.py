"""Model folders: safetensors by tensor name, checks against the spec, random weights."""
from .expected import expected_tensors, layer_tensors, probe_prefix
from .loader import check_store, load_weights
from .random_init import random_tensors, write_random_model
from .safetensors_io import SafetensorsFile, WeightError, WeightStore, write_safetensors

__all__ = ["expected_tensors", "layer_tensors", "probe_prefix", "check_store", "load_weights",
           "random_tensors", "write_random_model", "SafetensorsFile", "WeightError", "WeightStore",
           "write_safetensors"]
