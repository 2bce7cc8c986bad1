"""Reads a model folder's tensors against what the model spec expects.

Tensors are kept as stored: bfloat16 stays bfloat16 and float32 stays float32
(float16 is widened to float32, which is exact; float64 is narrowed to float32);
integer tables become int32. Every mismatch between the folder and the spec is
gathered into ONE error that lists missing tensors, unexpected tensors and wrong
shapes, so a broken checkpoint is diagnosed in one run. The reference fails on the
first missing name (src/io/safetensors.cpp:14-18) and checks shapes where a layer is
built (src/models/lfm3/lfm3_decoder.cpp:100-103).
"""
from __future__ import annotations

import warnings
from typing import Dict, List

import torch

from ..config.spec import ModelSpec
from .expected import expected_tensors, probe_prefix
from .safetensors_io import WeightError, WeightStore

_MAX_LISTED = 12


def _listing(items: List[str]) -> str:
    shown = items[:_MAX_LISTED]
    more = len(items) - len(shown)
    return ", ".join(shown) + (f", ... and {more} more" if more > 0 else "")


def check_store(spec: ModelSpec, store: WeightStore) -> str:
    """Raises WeightError unless the store holds exactly the spec's tensors with the
    spec's shapes. Returns the model prefix found."""
    prefix = probe_prefix(spec, store.names())
    expected = expected_tensors(spec, prefix)
    missing = [n for n in expected if n not in store]
    # Under a wrapper's prefix (a checkpoint that holds other towers beside the text decoder) only names under
    # that prefix, and the head's, are this model's to judge: the rest is read by name and left alone, as the
    # reference does (src/io/safetensors.cpp:14-18). Under the plain prefix every stray tensor is named.
    wrapped = prefix != spec.prefixes[-1]
    unexpected = [n for n in store.names() if n not in expected
                  and (not wrapped or n.startswith(prefix) or n == spec.names["head"])]
    wrong = [f"{n} is {list(store.shape(n))}, expected {list(ts.shape)}"
             for n, ts in expected.items() if n in store and tuple(store.shape(n)) != tuple(ts.shape)]
    bad_dtype = [f"{n} is {store.dtype(n)}" for n in expected
                 if n in store and not (store.dtype(n).is_floating_point or
                                        store.dtype(n) in (torch.int32, torch.int64, torch.int16, torch.int8,
                                                           torch.uint8))]
    if missing or unexpected or wrong or bad_dtype:
        parts = [f"'{store.where}' does not fit the {spec.arch} configuration:"]
        if missing:
            parts.append(f"  missing ({len(missing)}): {_listing(missing)}")
        if unexpected:
            parts.append(f"  unexpected ({len(unexpected)}): {_listing(unexpected)}")
        if wrong:
            parts.append(f"  wrong shape ({len(wrong)}): {_listing(wrong)}")
        if bad_dtype:
            parts.append(f"  unsupported dtype ({len(bad_dtype)}): {_listing(bad_dtype)}")
        raise WeightError("\n".join(parts))
    return prefix


def _as_kept(t: torch.Tensor) -> torch.Tensor:
    if t.dtype in (torch.bfloat16, torch.float32, torch.int32):
        return t
    if t.dtype in (torch.float16, torch.float64):
        return t.to(torch.float32)
    if not t.dtype.is_floating_point:
        return t.to(torch.int32)
    return t.to(torch.float32)


def load_weights(spec: ModelSpec, folder: str) -> Dict[str, torch.Tensor]:
    """{name without the model prefix: CPU tensor as stored}; the untied head keeps its
    own name."""
    store = WeightStore.open_dir(folder)
    prefix = check_store(spec, store)
    out: Dict[str, torch.Tensor] = {}
    with warnings.catch_warnings():
        warnings.simplefilter("ignore", UserWarning)   # views of a read-only mapping
        for name in expected_tensors(spec, prefix):
            key = name[len(prefix):] if name.startswith(prefix) else name
            out[key] = _as_kept(store.get(name))
    return out
