"""Random-weights mode: a model folder from a configuration and a seed.

Writes `config.json` and `model.safetensors`. Tensors are drawn in the order of
weights.expected.expected_tensors (embedding, final norm, head, then each layer's
tensors in the order its parts declare them); tensor number i uses the counter-based
generator Philox keyed by (seed, i), so a tensor's values do not depend on the others'
sizes. Matrices and tables are N(0, std) with std from the configuration
(`initializer_range`) unless given; norm weights are 1, or uniform in `norm_range`
when a test wants a skipped norm to show; biases are N(0, std).

The reference has random checkpoints only in its tests
(tests/unit/model/tiny_checkpoints.h:52-80); the layout written here is the one its
loader reads (src/models/lfm3/lfm3_decoder.cpp:14-19).
"""
from __future__ import annotations

import json
import os
from typing import Dict, Iterator, Optional, Tuple

import numpy as np
import torch

from .expected import expected_tensors
from .safetensors_io import write_safetensors

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16,
           "f32": torch.float32}


def random_tensors(spec, seed: int, dtype: str = "bfloat16", std: Optional[float] = None,
                   norm_range: Optional[Tuple[float, float]] = None,
                   scale: Optional[Dict[str, float]] = None) -> Iterator[Tuple[str, torch.Tensor]]:
    """Yields (full name, CPU tensor). `scale` multiplies tensors whose name ends with a
    given suffix (tests use it to make one part's effect stand out)."""
    tdtype = _DTYPES[dtype]
    sigma = spec.init_std if std is None else std
    for i, (name, ts) in enumerate(expected_tensors(spec).items()):
        rng = np.random.Generator(np.random.Philox(key=[seed & (2 ** 64 - 1), i]))
        if ts.init == "ones":
            if norm_range is None:
                a = np.ones(ts.shape, dtype=np.float32)
            else:
                a = rng.uniform(norm_range[0], norm_range[1], size=ts.shape).astype(np.float32)
        elif ts.init == "zeros":
            a = np.zeros(ts.shape, dtype=np.float32)
        else:
            a = rng.standard_normal(size=ts.shape, dtype=np.float32) * np.float32(sigma)
        if scale:
            for suffix, factor in scale.items():
                if name.endswith(suffix):
                    a = a * np.float32(factor)
        t = torch.from_numpy(np.ascontiguousarray(a))
        # vectors (norm weights, taps' biases) are stored in float32 even beside bfloat16 matrices
        yield name, (t if ts.role == "vector" else t.to(tdtype))


def write_random_model(folder: str, config, seed: int, dtype: str = "bfloat16",
                       std: Optional[float] = None,
                       norm_range: Optional[Tuple[float, float]] = None,
                       scale: Optional[Dict[str, float]] = None,
                       generation: Optional[dict] = None) -> str:
    """`config` is a typed configuration (to_json(), model_spec()). Returns `folder`."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config.to_json(), f, indent=1)
    if generation is not None:
        with open(os.path.join(folder, "generation_config.json"), "w", encoding="utf-8") as f:
            json.dump(generation, f, indent=1)
    spec = config.model_spec()
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      random_tensors(spec, seed, dtype, std, norm_range, scale),
                      metadata={"format": "pt", "seed": str(seed)})
    return folder
