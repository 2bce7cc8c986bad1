"""Sampling parameters and the device sampler."""
from .params import (FINISH_CANCELLED, FINISH_ERROR, FINISH_LENGTH, FINISH_STOP, GenerateRequest,
                     GenerateResult, GenerateStats, SamplingParams, TokenCallback, read_generation_defaults)

__all__ = ["FINISH_CANCELLED", "FINISH_ERROR", "FINISH_LENGTH", "FINISH_STOP", "GenerateRequest",
           "GenerateResult", "GenerateStats", "SamplingParams", "TokenCallback", "read_generation_defaults"]
